"""Tensor-parallel decoder layer on 2 GPUs (one process per GPU) against the unsharded CPU oracle:
the partial sums of the output projection and of the down projection exchanged inside the kernels
over peer memory ("peer"), or with an NCCL all-reduce ("nccl").  Skipped on a machine with one GPU."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


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
    if B > 1:
        seqlens[1] = ctx - 3
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    return w, x, kc, vc, seqlens, cos, sin


def _worker(rank, world, port, shape_name, B, ctx, exchange, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flashsvd_b200 import tensor_parallel as TP

        shape = getattr(O, shape_name)
        S_max = ctx + 4
        w, x, kc, vc, seqlens, cos, sin = _case(shape, B, ctx, S_max, seed=3)
        ws = TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=rank, world=world)
        ex = TP.PeerExchange(rank=rank, world=world, max_rows=B, d=shape.d) if exchange == "peer" else None
        layer = TP.TPDecodeLayer(ws, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=rank, world=world, batch=B, S_max=S_max,
                                 eps=shape.eps, device=dev, exchange=ex)
        hk = shape.Hk // world
        layer.k_cache.copy_(kc[:, :, rank * hk:(rank + 1) * hk])
        layer.v_cache.copy_(vc[:, :, rank * hk:(rank + 1) * hk])
        xd, sl, cd, sd = x.to(dev), seqlens.to(dev), cos.to(dev), sin.to(dev)
        torch.cuda.synchronize()
        dist.barrier()          # the ranks start together: a wait for a peer is bounded (about 2 s)
        y = layer.forward(xd, sl, cd, sd).clone()
        # the same token again (both parities of the exchange buffers): the same bits
        for _ in range(3):
            y2 = layer.forward(xd, sl, cd, sd)
        torch.cuda.synchronize()
        assert layer.ws.status() == 0
        assert torch.equal(y, y2)
        # every rank holds the same output bits
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        assert all(torch.equal(ys[0], t) for t in ys)
        if rank == 0:
            kco, vco = kc.clone(), vc.clone()
            ref = O.decode_layer(shape, w, x, kco, vco, seqlens, cos, sin)
            err = float((y.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())
            kerr = float((layer.k_cache.float().cpu() - kco[:, :, :hk].float()).abs().max() / kco.float().abs().max())
            out.put((err, kerr))
        if ex is not None:
            ex.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape_name,B,ctx,exchange", [("TINY_GQA", 2, 30, "nccl"), ("LLAMA70B_SVD40", 8, 200, "nccl"),
                                                        ("TINY_GQA", 2, 30, "peer"), ("LLAMA70B_SVD40", 8, 200, "peer"),
                                                        ("TINY_GQA", 24, 50, "peer")])
def test_tp_layer_on_two_gpus_matches_the_unsharded_oracle(shape_name, B, ctx, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mpc = mp.get_context("spawn")
    out = mpc.Queue()
    port = 29600 + os.getpid() % 2000
    procs = [mpc.Process(target=_worker, args=(r, 2, port, shape_name, B, ctx, exchange, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    err, kerr = out.get(timeout=5)
    print(f"{shape_name} B={B} {exchange}: layer output rel_linf {err:.3e}, appended keys {kerr:.3e}")
    assert err <= 2e-2 and kerr <= 2e-2


def _model_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from flashsvd_b200 import synthetic
        from flashsvd_b200 import tensor_parallel as TP

        shape = synthetic.ModelShape(d=256, H=8, Hk=2, Dh=64, I=640, Rq=96, Rk=32, Rv=32, Ro=96, Rg=120, Ru=120, Rd=120,
                                     vocab=384, n_layers=3)
        toks = {}
        for use_graph in (False, True):
            m = TP.random_tp_model(shape, rank=rank, world=world, device=dev, batch=8, ctx=17, max_new=12, seed=1,
                                   use_graph=use_graph, exchange="peer")
            seen = []
            for _ in range(6):
                m.step(1)
                seen.append(m.tokens.clone())
            torch.cuda.synchronize()
            assert m.status() == 0
            toks[use_graph] = torch.stack(seen)
            m.close()
        # eager launches and the replayed CUDA graph give the same tokens; every rank holds the same tokens
        assert torch.equal(toks[False], toks[True])
        both = [torch.empty_like(toks[True]) for _ in range(world)]
        dist.all_gather(both, toks[True])
        assert all(torch.equal(both[0], t) for t in both)
        if rank == 0:
            out.put(toks[True].cpu().tolist())   # plain lists: nothing shared outlives the worker
    finally:
        dist.destroy_process_group()


def test_tp_model_with_the_peer_exchange_steps_on_two_gpus():
    """Three layers, six tokens: eager launches against the CUDA-graph replay, rank against rank."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mpc = mp.get_context("spawn")
    out = mpc.Queue()
    port = 29600 + (os.getpid() + 7) % 2000
    procs = [mpc.Process(target=_model_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    toks = out.get(timeout=5)
    assert len(toks) == 6 and len(toks[0]) == 8
