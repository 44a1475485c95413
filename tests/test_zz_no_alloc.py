"""fsvd_lowrank_proj_static (built-in scratch, no device allocation) against fsvd_lowrank_proj
(caller workspace), both through the C ABI.  The file name sorts last so that it also runs after
every other GPU test has used the library in the same process."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, x, v, u, res, y):
    B, d_in = x.shape
    R, d_out = v.shape[0], u.shape[0]
    from flashsvd_b200 import _lib

    code = _lib.DTYPE_BF16 if x.dtype == torch.bfloat16 else _lib.DTYPE_F32
    return lib.fsvd_lowrank_proj_static(x.data_ptr(), v.data_ptr(), u.data_ptr(),
                                        res.data_ptr() if res is not None else None, y.data_ptr(), B, d_in, R,
                                        d_out, code, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype,B,d_in,R,d_out", [(torch.bfloat16, 1, 4096, 1024, 4096),
                                                 (torch.float32, 2, 264, 88, 520),
                                                 (torch.bfloat16, 8, 11008, 1024, 4096),
                                                 # few rank rows and a long input: the K-segment plan is
                                                 # what decides the summation order here
                                                 (torch.bfloat16, 1, 8192, 88, 512)])
def test_static_scratch_matches_workspace_variant(dtype, B, d_in, R, d_out):
    from flashsvd_b200 import _lib, ops

    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(B * 1000 + R)
    v = (torch.randn(R, d_in, device=dev, generator=g) / d_in ** 0.5).to(dtype)
    u = (torch.randn(d_out, R, device=dev, generator=g) / R ** 0.5).to(dtype)
    dims = ops.make_dims(dtype=dtype, B=B, d=d_out, Ro=R)
    ws = ops.make_workspace(dims, dev)
    # two calls in a row on the shared scratch, different inputs, the second with a residual
    for it in range(2):
        x = torch.randn(B, d_in, device=dev, generator=g).to(dtype)
        res = torch.randn(B, d_out, device=dev, generator=g).to(dtype) if it else None
        want = ops.lowrank_proj(x, v, u, ws, residual=res)
        got = torch.full_like(want, float("nan"))
        _lib.check(_call_static(lib, x, v, u, res, got))
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        ref = torch.nn.functional.linear(torch.nn.functional.linear(x.float(), v.float()).to(dtype).float(), u.float())
        if res is not None:
            ref = ref + res.float()
        err = float((got.float() - ref).abs().max() / ref.abs().max())
        assert err <= (2e-2 if dtype == torch.bfloat16 else 2e-5)
    assert ws.status() == 0
    st = C.c_int(-1)
    _lib.check(lib.fsvd_static_status(C.byref(st), 0))
    assert st.value == 0


def test_static_scratch_rejects_oversize():
    from flashsvd_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda:0")
    B, d_in, R, d_out = 2, 64, 8192, 64  # B * R = 16384 > 8192
    x = torch.zeros(B, d_in, device=dev)
    v = torch.zeros(R, d_in, device=dev)
    u = torch.zeros(d_out, R, device=dev)
    y = torch.zeros(B, d_out, device=dev)
    before = int(lib.fsvd_launch_count())
    rc = _call_static(lib, x, v, u, None, y)
    assert rc == -4
    assert b"built-in scratch" in lib.fsvd_last_error_string()
    assert int(lib.fsvd_launch_count()) == before
    with pytest.raises(ValueError):
        _lib.check(rc)
