"""What happens when something goes wrong on the device: a wait that runs out, a token past the
end of the cache, a change of the launch geometry between two launches on one workspace.  None of
these cases faults or hangs anything: the waits are bounded by design and the test only makes one
run out."""
import ctypes as C

import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu

DEFAULT_WAIT = 4_000_000_000


def _lowrank_case(dev, dtype=torch.bfloat16, B=2, d_in=1024, R=256, d_out=768, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(B, d_in, device=dev, generator=g).to(dtype)
    v = (torch.randn(R, d_in, device=dev, generator=g) / d_in ** 0.5).to(dtype)
    u = (torch.randn(d_out, R, device=dev, generator=g) / R ** 0.5).to(dtype)
    lin = torch.nn.functional.linear
    ref = lin(lin(x.float(), v.float()).to(dtype).float(), u.float())
    return x, v, u, ref


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


def test_wait_that_runs_out_is_reported_and_the_workspace_recovers():
    """A grid barrier nobody arrives at: every CTA gives up after the budget (2e6 clocks, about a
    millisecond), the launch ends by itself, the status word says which wait and which stage, and
    the same workspace then runs a normal launch correctly."""
    from flashsvd_b200 import _lib, ops

    lib = _lib.load()
    dev = torch.device("cuda:0")
    dims = ops.make_dims(dtype=torch.bfloat16, B=2, d=768, Ro=256)
    ws = ops.make_workspace(dims, dev)
    x, v, u, ref = _lowrank_case(dev)
    try:
        ops.set_wait_limit(2_000_000)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        _lib.check(lib.fsvd_selftest_wait_timeout(ws.ptr, ws.nbytes, torch.cuda.current_stream().cuda_stream))
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0   # ms: ended by the budget, far from any watchdog
        assert ws.raw_status() == 1          # a grid-barrier wait ran out
        with pytest.raises(_lib.FsvdError, match="stage 0"):
            ws.status()
        # sticky until cleared; a launch on the flagged workspace still runs and still ends
        ops.set_wait_limit(DEFAULT_WAIT)
        y = ops.lowrank_proj(x, v, u, ws)
        torch.cuda.synchronize()
        assert ws.raw_status() == 1
        assert _rel(y, ref) <= 2e-2
        ws.clear_status()
        y = ops.lowrank_proj(x, v, u, ws)
        assert ws.status() == 0
        assert _rel(y, ref) <= 2e-2
    finally:
        ops.set_wait_limit(DEFAULT_WAIT)


def test_wait_limit_argument_is_checked():
    from flashsvd_b200 import ops

    with pytest.raises(ValueError):
        ops.set_wait_limit(10)


@pytest.mark.parametrize("grids", [(0, 64, 0), (37, 148, 5)])
def test_launch_geometry_may_change_between_launches_on_one_workspace(grids):
    """The barrier count starts at zero in every launch, so two launches with different grids can
    follow each other on one workspace (and on the built-in scratch)."""
    from flashsvd_b200 import ops

    dev = torch.device("cuda:0")
    dims = ops.make_dims(dtype=torch.bfloat16, B=2, d=768, Ro=256)
    ws = ops.make_workspace(dims, dev)
    try:
        for i, g in enumerate(grids):
            ops.set_launch_config(grid=g)
            x, v, u, ref = _lowrank_case(dev, seed=i)
            y = ops.lowrank_proj(x, v, u, ws)
            ys = ops.lowrank_proj_static(x, v, u)
            torch.cuda.synchronize()
            assert _rel(y, ref) <= 2e-2
            assert torch.equal(y, ys)
        assert ws.status() == 0
    finally:
        ops.set_launch_config()


def _tiny_engine(dev, S_max):
    from flashsvd_b200 import engine, packing

    shape, dtype = O.TINY, torch.float32
    w = O.make_model_weights(shape, seed=1, dtype=dtype)
    layers = [packing.pack_layer(lw, device=dev, dtype=dtype) for lw in w["layers"]]
    eng = engine.DecodeEngine(layers=layers, embed=w["embed"].to(dev), final_norm=w["norm"].to(dev),
                              lm_head=w["lm_head"].to(dev), num_heads=shape.H, num_kv_heads=shape.Hk,
                              head_dim=shape.Dh, batch_size=1, max_cache_len=S_max, rope_theta=shape.theta,
                              eps=shape.eps, max_steps=64)
    return eng, shape, w


def test_full_cache_raises_index_error_on_the_host_and_flags_on_the_device():
    """The reference's dense cache raises IndexError when a token does not fit
    (runtime/cache/attn_dense_kv.py:295-298).  The engine raises before the launch; a caller of the
    C ABI that steps anyway gets status 4 (FSVD_ERR_CACHE_FULL), and the cache is left untouched."""
    from flashsvd_b200 import _lib

    dev = torch.device("cuda:0")
    S_max = 8
    eng, shape, w = _tiny_engine(dev, S_max)
    prompt = torch.randint(0, shape.vocab, (1, 6), generator=torch.Generator().manual_seed(2))
    eng.prefill(prompt)
    eng.step(2)                       # positions 6 and 7: the cache is now full
    assert eng.status() == 0
    ref, _, _ = O.greedy_decode(shape, w, prompt, 3)
    assert eng.last_tokens(3)[:, 0].tolist() == ref[0].tolist()
    with pytest.raises(IndexError):
        eng.step(1)
    assert eng.status() == 0          # nothing was launched
    # the C ABI itself: one more step at position 8 = S_max
    k_before = [t.clone() for t in eng.key_cache]
    v_before = [t.clone() for t in eng.value_cache]
    _lib.check(eng.lib.fsvd_model_step(eng.handle, 1, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    with pytest.raises(IndexError, match="S_max"):
        eng.status()
    for k, v, kb, vb in zip(eng.key_cache, eng.value_cache, k_before, v_before):
        assert torch.equal(k, kb) and torch.equal(v, vb)
    # reset and generate again from a clean state
    _lib.check(eng.lib.fsvd_model_reset_sync(eng.handle, torch.cuda.current_stream().cuda_stream))
    eng.reset()
    eng.prefill(prompt)
    eng.step(1)
    assert eng.status() == 0
    assert eng.last_tokens(2)[:, 0].tolist() == ref[0].tolist()[:2]
    eng.close()
