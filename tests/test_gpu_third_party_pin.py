"""Pins the attention half of the path to the third-party arithmetic the reference calls.

The reference's decode attention is flash-attn's ``flash_attn_with_kvcache`` (rotary on q and the
new key at position cache_seqlens, append of k / v, causal softmax(q K^T / sqrt(Dh)) V with GQA;
call site runtime/attn/decode_registry.py:177-211, pinned flash-attn 2.8.3).  The same wheel is in
this image, so the library function itself is run here on the same inputs as
``fsvd_qkv_rope_append`` + ``fsvd_flash_decode``.  The reference's own Python files are not on the
GPU machine and are not needed: the call below passes the arguments its call site passes
(rotary_interleaved=False, causal=True, cos / sin tables [S, Dh/2]).

If the wheel cannot run on this GPU the test is skipped with the library's own message.
"""
import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max())


@pytest.mark.parametrize("shape_name,B,ctx", [("TINY_GQA", 2, 37), ("TINY", 1, 300)])
def test_flash_attn_with_kvcache_agrees(shape_name, B, ctx):
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as e:  # pragma: no cover - depends on the image
        pytest.skip(f"flash_attn cannot be imported: {e}")
    from flashsvd_b200 import ops, packing

    dev = torch.device("cuda:0")
    dtype = torch.bfloat16
    shape = getattr(O, shape_name)
    gen = torch.Generator().manual_seed(11)
    w = O.make_layer_weights(shape, gen, dtype)
    d = packing.pack_layer(w, device=dev, dtype=dtype)
    S_max = ctx + 8
    H, Hk, Dh = shape.H, shape.Hk, shape.Dh
    x = torch.randn(B, shape.d, generator=gen).to(dtype).to(dev)
    kc = torch.zeros(B, S_max, Hk, Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    kc[:, :ctx] = torch.randn(B, ctx, Hk, Dh, generator=gen).to(dtype)
    vc[:, :ctx] = torch.randn(B, ctx, Hk, Dh, generator=gen).to(dtype)
    seq = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    cos, sin = O.rope_tables(S_max, Dh, shape.theta, dtype)
    cos, sin = cos.to(dev), sin.to(dev)

    # this library: rank projection + lift + rotary + append, then attention over ctx + 1 keys
    dims = ops.make_dims(dtype=dtype, B=B, d=shape.d, H=H, Hk=Hk, Dh=Dh, I=shape.I, Rq=shape.Rq, Rk=shape.Rk,
                         Rv=shape.Rv, Ro=shape.Ro, Rg=shape.Rg, Ru=shape.Ru, Rd=shape.Rd, S_max=S_max)
    ws = ops.make_workspace(dims, dev)
    k1, v1 = kc.to(dev), vc.to(dev)
    qkv_v = torch.cat([w["q_v"], w["k_v"], w["v_v"]], 0).to(dev).contiguous()
    q_rot = ops.qkv_rope_append(x, qkv_v, d["q_u"], d["k_u"], d["v_u"], cos, sin, k1, v1, seq, ws,
                                num_heads=H, num_kv_heads=Hk, head_dim=Dh, ranks=(shape.Rq, shape.Rk, shape.Rv))
    out1 = ops.flash_decode(q_rot, k1, v1, seq, ws, seqlen_add=1)
    torch.cuda.synchronize()
    assert ws.status() == 0

    # flash-attn: the un-rotated q / k / v of the same token from the PyTorch low-rank path
    lin = torch.nn.functional.linear
    wd = {k: v.to(dev) for k, v in w.items()}
    q = lin(lin(x, wd["q_v"]), wd["q_u"]).view(B, 1, H, Dh)
    k = lin(lin(x, wd["k_v"]), wd["k_u"]).view(B, 1, Hk, Dh)
    v = lin(lin(x, wd["v_v"]), wd["v_u"]).view(B, 1, Hk, Dh)
    k2, v2 = kc.to(dev), vc.to(dev)
    try:
        out2 = flash_attn_with_kvcache(q, k2, v2, k=k, v=v, rotary_cos=cos, rotary_sin=sin, cache_seqlens=seq,
                                       softmax_scale=Dh ** -0.5, causal=True, rotary_interleaved=False)
        torch.cuda.synchronize()
    except RuntimeError as e:  # pragma: no cover - depends on the wheel's architectures
        pytest.skip(f"flash_attn_with_kvcache does not run on this GPU: {e}")
    # appended rows: rotated key and value of the new token at position ctx
    assert _rel(k1[:, ctx], k2[:, ctx]) <= 2e-2
    assert _rel(v1[:, ctx], v2[:, ctx]) <= 2e-2
    assert torch.equal(k1[:, :ctx], k2[:, :ctx]) and torch.equal(k1[:, ctx + 1:], k2[:, ctx + 1:])
    assert _rel(out1.reshape(B, -1), out2.reshape(B, -1)) <= 2e-2
