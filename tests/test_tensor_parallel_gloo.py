"""Tensor-parallel partitioning on CPU (gloo, world size 2): the sharded oracle, summed over the
ranks, equals the unsharded oracle layer; the shard bookkeeping is exact."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import lowrank_llama as O


def test_shards_partition_every_sharded_factor_exactly():
    from flashsvd_b200 import tensor_parallel as TP

    shape = O.TINY_GQA
    w = O.make_layer_weights(shape, torch.Generator().manual_seed(0), torch.float32)
    shards = [TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=r, world=2) for r in range(2)]
    for name in TP.ROW_SHARDED:
        assert torch.equal(torch.cat([s[name] for s in shards], 0), w[name])
    for name in TP.COL_SHARDED:
        assert torch.equal(torch.cat([s[name] for s in shards], 1), w[name])
    for name in ("q_v", "k_v", "v_v", "o_u", "gate_v", "up_v", "down_u", "ln1", "ln2"):
        assert torch.equal(shards[0][name], w[name]) and torch.equal(shards[1][name], w[name])
    with pytest.raises(ValueError):
        TP.shard_ranges(shape.H, shape.Hk, shape.Dh, shape.I, 0, 3)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashsvd_b200 import tensor_parallel as TP
        from oracle import tensor_parallel as OTP

        shape, B, ctx, S_max = O.TINY_GQA, 3, 9, 16
        gen = torch.Generator().manual_seed(1)
        w = O.make_layer_weights(shape, gen, torch.float32)
        x = torch.randn(B, shape.d, generator=gen)
        kc = torch.zeros(B, S_max, shape.Hk, shape.Dh)
        vc = torch.zeros_like(kc)
        kc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen)
        vc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen)
        seqlens = torch.tensor([ctx, ctx - 2, ctx - 5], dtype=torch.int32)
        cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, torch.float32)
        ref = O.decode_layer(shape, w, x, kc.clone(), vc.clone(), seqlens, cos, sin)
        hk = shape.Hk // world
        kcs, vcs = kc[:, :, rank * hk:(rank + 1) * hk].clone(), vc[:, :, rank * hk:(rank + 1) * hk].clone()
        ws = TP.shard_layer_weights(w, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, rank=rank, world=world)

        def allreduce(t):
            t = t.clone()
            dist.all_reduce(t)
            return t

        got = OTP.decode_layer_shard(shape, ws, x, kcs, vcs, seqlens, cos, sin, rank=rank, world=world, allreduce=allreduce)
        err = float((got - ref).abs().max() / ref.abs().max())
        if rank == 0:
            out.put(err)
    finally:
        dist.destroy_process_group()


def test_sharded_oracle_sums_to_the_unsharded_layer():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(timeout=5) <= 1e-5     # fp32: summation order only
