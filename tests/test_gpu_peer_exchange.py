"""The in-kernel exchange of the tensor-parallel layer on ONE GPU: the pushing GEMM epilogue, the
flags, the sequence numbers and the reducing kernel, with the other rank's partial sums and flags
written by the host beforehand (kernels that wait for each other never run side by side on one
GPU); and the bounded wait: a peer that never posts ends in an error status, not a hang."""
import pytest
import torch
import torch.nn.functional as F

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(shape, B, ctx, S_max, seed):
    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(seed)
    w = O.make_layer_weights(shape, gen, dtype)
    x = torch.randn(B, shape.d, generator=gen).to(dtype)
    kc = torch.zeros(B, S_max, shape.Hk, shape.Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    kc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen).to(dtype)
    vc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen).to(dtype)
    seqlens = torch.full((B,), ctx, dtype=torch.int32)
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    return w, x, kc, vc, seqlens, cos, sin


def _oracle_partials(shape, shards, x, kcs, vcs, seqlens, cos, sin):
    """Both exchanges of a layer on the CPU: per-rank partial sums of the o projection, the full h,
    per-rank partial sums of the down projection, the full layer output."""
    world, B = len(shards), x.shape[0]
    Hl, Hkl, Dh = shape.H // world, shape.Hk // world, shape.Dh
    parts = []
    for r, w in enumerate(shards):
        xn = O.rmsnorm(x, w["ln1"], shape.eps)
        q = F.linear(F.linear(xn, w["q_v"]), w["q_u"]).view(B, Hl, Dh)
        k = F.linear(F.linear(xn, w["k_v"]), w["k_u"]).view(B, Hkl, Dh)
        v = F.linear(F.linear(xn, w["v_v"]), w["v_u"]).view(B, Hkl, Dh)
        attn = torch.empty(B, Hl * Dh, dtype=x.dtype)
        for b in range(B):
            pos = int(seqlens[b])
            c, s = cos[pos].unsqueeze(0), sin[pos].unsqueeze(0)
            kcs[r][b, pos] = O.rotate_half_apply(k[b], c, s)
            vcs[r][b, pos] = v[b]
            attn[b] = O.attend(O.rotate_half_apply(q[b], c, s), kcs[r][b, : pos + 1], vcs[r][b, : pos + 1]).reshape(-1)
        parts.append(O.lowrank(attn, w["o_v"], w["o_u"]))
    h = (x.float() + sum(p.float() for p in parts)).to(x.dtype)
    parts2 = []
    for w in shards:
        hn = O.rmsnorm(h, w["ln2"], shape.eps)
        act = F.silu(F.linear(F.linear(hn, w["gate_v"]), w["gate_u"])) * F.linear(F.linear(hn, w["up_v"]), w["up_u"])
        parts2.append(F.linear(F.linear(act, w["down_v"]), w["down_u"]))
    y = (h.float() + sum(p.float() for p in parts2)).to(x.dtype)
    return parts, h, parts2, y


def _region_views(buf, lay, world):
    flags = buf[lay["flags"]: lay["flags"] + 2 * world * lay["flag_cap"] * 4].view(torch.int32).view(2, world, lay["flag_cap"])
    slots = buf[lay["slots"]: lay["slots"] + 2 * world * lay["slot_bytes"]].view(2, world, lay["slot_bytes"])
    return flags, slots


def _slot_rows(slots, parity, src, B, d):
    return slots[parity, src, : B * d * 2].view(torch.bfloat16).view(B, d)


@pytest.mark.parametrize("shape_name,B,ctx,world", [("TINY_GQA", 3, 20, 1), ("TINY_GQA", 8, 20, 2), ("TINY_GQA", 16, 40, 2)])
def test_tp_layer_rank0_with_the_peer_preposted(shape_name, B, ctx, world):
    from flashsvd_b200 import tensor_parallel as TP

    shape = getattr(O, shape_name)
    S_max = ctx + 4
    w, x, kc, vc, seqlens, cos, sin = _case(shape, B, ctx, S_max, seed=11)
    shards = [TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=r, world=world) for r in range(world)]
    hk = shape.Hk // world
    kcs = [kc[:, :, r * hk:(r + 1) * hk].clone() for r in range(world)]
    vcs = [vc[:, :, r * hk:(r + 1) * hk].clone() for r in range(world)]
    kc0, vc0 = kcs[0].clone(), vcs[0].clone()
    parts, h, parts2, y_ref = _oracle_partials(shape, shards, x, kcs, vcs, seqlens, cos, sin)

    lay = TP.region_layout(world, B, shape.d)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=DEV) for _ in range(world)]
    ex = TP.PeerExchange(rank=0, world=world, max_rows=B, d=shape.d, regions=[b.data_ptr() for b in bufs])
    assert ex.nbytes == lay["total"]
    flags0, slots0 = _region_views(bufs[0], lay, world)
    if world == 2:
        # what rank 1 would have stored into rank 0's region: exchange 1 (parity 1), exchange 2 (parity 0)
        _slot_rows(slots0, 1, 1, B, shape.d).copy_(parts[1].to(DEV))
        _slot_rows(slots0, 0, 1, B, shape.d).copy_(parts2[1].to(DEV))
        flags0[1, 1, :] = 1
        flags0[0, 1, :] = 2
    layer = TP.TPDecodeLayer(shards[0], H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=world, batch=B, S_max=S_max,
                             eps=shape.eps, device=DEV, exchange=ex)
    layer.k_cache.copy_(kc0)
    layer.v_cache.copy_(vc0)
    y = layer.forward(x.to(DEV), seqlens.to(DEV), cos.to(DEV), sin.to(DEV))
    torch.cuda.synchronize()
    assert layer.ws.status() == 0
    scale = float(y_ref.float().abs().max())
    err = float((y.float().cpu() - y_ref.float()).abs().max()) / scale
    kerr = float((layer.k_cache.float().cpu() - kcs[0].float()).abs().max() / kcs[0].float().abs().max())
    print(f"{shape_name} B={B} world={world}: rank 0 layer output rel_linf {err:.3e}, keys {kerr:.3e}")
    assert err <= 2e-2 and kerr <= 2e-2
    # the partial sums rank 0 pushed: the same bytes in every region, close to the oracle's
    for parity, ref in ((1, parts[0]), (0, parts2[0])):
        mine = _slot_rows(slots0, parity, 0, B, shape.d)
        perr = float((mine.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())
        assert perr <= 2e-2, perr
        for b in bufs[1:]:
            _, slots_q = _region_views(b, lay, world)
            assert torch.equal(_slot_rows(slots_q, parity, 0, B, shape.d), mine)
    # one flag per CTA of the pushing GEMM in every region, and the sequence number moved on by 2
    for b in bufs:
        fl, _ = _region_views(b, lay, world)
        assert int((fl[1, 0] == 1).sum()) >= 1 and int((fl[0, 0] == 2).sum()) >= 1
    assert int(bufs[0][:4].view(torch.int32)[0]) == 3
    ex.close()


def test_a_peer_that_never_posts_ends_in_an_error_status():
    from flashsvd_b200 import ops
    from flashsvd_b200 import tensor_parallel as TP

    shape, B, ctx, world = O.TINY_GQA, 4, 12, 2
    S_max = ctx + 4
    w, x, kc, vc, seqlens, cos, sin = _case(shape, B, ctx, S_max, seed=5)
    sh = TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=world)
    lay = TP.region_layout(world, B, shape.d)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=DEV) for _ in range(world)]
    ex = TP.PeerExchange(rank=0, world=world, max_rows=B, d=shape.d, regions=[b.data_ptr() for b in bufs])
    ops.set_wait_limit(2_000_000)          # about a millisecond of SM clocks
    try:
        layer = TP.TPDecodeLayer(sh, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=world, batch=B, S_max=S_max,
                                 eps=shape.eps, device=DEV, exchange=ex)
        y = layer.forward(x.to(DEV), seqlens.to(DEV), cos.to(DEV), sin.to(DEV))
        torch.cuda.synchronize()           # returns: both waits gave up
        assert layer.ws.raw_status() == 8
        with pytest.raises(RuntimeError, match="device wait ran out"):
            layer.ws.status()
        assert torch.isfinite(y.float()).all()
        layer.ws.clear_status()
        torch.cuda.synchronize()
        assert layer.ws.raw_status() == 0
        assert int(bufs[0][:4].view(torch.int32)[0]) == 3   # the exchange moved on all the same
    finally:
        ops.set_wait_limit(4_000_000_000)
        ex.close()


def test_norms_of_the_neighbouring_layers_fused_into_the_exchange():
    """x_norm (input already normalised by the layer before) and next_norm_w (the finishing kernel
    also writes the next layer's normalised input) against the plain call."""
    from flashsvd_b200 import tensor_parallel as TP

    shape, B, ctx, world = O.TINY_GQA, 6, 25, 1
    S_max = ctx + 4
    w, x, kc, vc, seqlens, cos, sin = _case(shape, B, ctx, S_max, seed=21)
    sh = TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=world)
    sh["ln1"] = (1.0 + 0.1 * torch.randn(shape.d)).to(torch.bfloat16)
    lay = TP.region_layout(world, B, shape.d)
    buf = torch.zeros(lay["total"], dtype=torch.uint8, device=DEV)
    ex = TP.PeerExchange(rank=0, world=world, max_rows=B, d=shape.d, regions=[buf.data_ptr()])
    layer = TP.TPDecodeLayer(sh, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=world, batch=B, S_max=S_max,
                             eps=shape.eps, device=DEV, exchange=ex)
    layer.k_cache.copy_(kc)
    layer.v_cache.copy_(vc)
    xd, sl, cd, sd = x.to(DEV), seqlens.to(DEV), cos.to(DEV), sin.to(DEV)
    y_plain = layer.forward(xd, sl, cd, sd).clone()
    nw = (1.0 + 0.1 * torch.randn(shape.d)).to(torch.bfloat16).to(DEV)
    xn = O.rmsnorm(x, sh["ln1"], shape.eps).to(DEV)
    y = layer.forward(xd, sl, cd, sd, x_norm=xn, next_norm_w=nw)
    torch.cuda.synchronize()
    assert layer.ws.status() == 0
    assert rel(y, y_plain) <= 4e-3          # the CPU norm and the kernel's may round a value differently
    want = O.rmsnorm(y.cpu(), nw.cpu(), shape.eps)
    assert rel(layer.out_norm, want) <= 1e-2
    ex.close()


def rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max())


def test_exchange_trace_records_every_reduction():
    from flashsvd_b200 import tensor_parallel as TP

    shape, B, ctx = O.TINY_GQA, 4, 12
    S_max = ctx + 4
    w, x, kc, vc, seqlens, cos, sin = _case(shape, B, ctx, S_max, seed=9)
    sh = TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=1)
    lay = TP.region_layout(1, B, shape.d)
    buf = torch.zeros(lay["total"], dtype=torch.uint8, device=DEV)
    ex = TP.PeerExchange(rank=0, world=1, max_rows=B, d=shape.d, regions=[buf.data_ptr()])
    ex.start_trace(records=16)
    layer = TP.TPDecodeLayer(sh, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=0, world=1, batch=B, S_max=S_max,
                             eps=shape.eps, device=DEV, exchange=ex)
    for _ in range(3):
        layer.forward(x.to(DEV), seqlens.to(DEV), cos.to(DEV), sin.to(DEV))
    torch.cuda.synchronize()
    s = ex.trace_summary()
    assert s["exchanges"] == 6                       # two per layer call
    assert 0 <= s["wait_us_median"] < 1e4 and 0 < s["reduce_us_median"] < 1e4
    ex.close()
