"""Tensor-parallel decoder layer on 2 GPUs (one process per GPU, NCCL all-reduce of the partial
sums of the output projection and of the down projection) against the unsharded CPU oracle.
Skipped on a machine with one GPU."""
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


def _worker(rank, world, port, shape_name, B, ctx, out):
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
        layer = TP.TPDecodeLayer(ws, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=rank, world=world, batch=B, S_max=S_max,
                                 eps=shape.eps, device=dev)
        hk = shape.Hk // world
        layer.k_cache.copy_(kc[:, :, rank * hk:(rank + 1) * hk])
        layer.v_cache.copy_(vc[:, :, rank * hk:(rank + 1) * hk])
        y = layer.forward(x.to(dev), seqlens.to(dev), cos.to(dev), sin.to(dev))
        torch.cuda.synchronize()
        assert layer.ws.status() == 0
        if rank == 0:
            kco, vco = kc.clone(), vc.clone()
            ref = O.decode_layer(shape, w, x, kco, vco, seqlens, cos, sin)
            err = float((y.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())
            kerr = float((layer.k_cache.float().cpu() - kco[:, :, :hk].float()).abs().max() / kco.float().abs().max())
            out.put((err, kerr))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape_name,B,ctx", [("TINY_GQA", 2, 30), ("LLAMA70B_SVD40", 8, 200)])
def test_tp_layer_on_two_gpus_matches_the_unsharded_oracle(shape_name, B, ctx):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mpc = mp.get_context("spawn")
    out = mpc.Queue()
    port = 29600 + os.getpid() % 2000
    procs = [mpc.Process(target=_worker, args=(r, 2, port, shape_name, B, ctx, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    err, kerr = out.get(timeout=5)
    print(f"{shape_name} B={B}: layer output rel_linf {err:.3e}, appended keys {kerr:.3e}")
    assert err <= 2e-2 and kerr <= 2e-2
