"""Batch-partitioned decode across ranks (no data-path collective): the host logic that
bench.py --gpus N uses, run as two gloo ranks on CPU.  Every rank decodes its own sequences; the
only exchange is the timing reduction (max over ranks) and the token gather on the host."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashsvd_b200 import partition


def test_partition_covers_every_sequence_once():
    for n_seq in (1, 2, 7, 8, 32, 129):
        for world in (1, 2, 4, 8):
            parts = [partition.sequences_of_rank(n_seq, r, world) for r in range(world)]
            flat = [i for p in parts for i in p]
            assert sorted(flat) == list(range(n_seq))
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    with pytest.raises(ValueError):
        partition.sequences_of_rank(4, 2, 2)


def test_aggregate_throughput_is_units_over_slowest_rank():
    assert partition.aggregate_tokens_per_s([32, 32], [100.0, 125.0]) == pytest.approx(64 / 0.125)
    assert partition.aggregate_tokens_per_s([10], [50.0]) == pytest.approx(200.0)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = partition.sequences_of_rank(5, rank, world)
        # stand-in for the decode: token ids derived from the sequence index
        tokens = {i: [i * 10 + t for t in range(3)] for i in mine}
        ms = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
        slowest = partition.max_over_ranks(ms)
        gathered = partition.gather_tokens(tokens, n_seq=5)
        total = partition.sum_over_ranks(torch.tensor([3.0 * len(mine)], dtype=torch.float64))
        if rank == 0:
            out.put((float(slowest), gathered, float(total)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_share_a_batch():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    slowest, gathered, total = out.get()
    assert slowest == 15.0
    assert gathered == [[i * 10 + t for t in range(3)] for i in range(5)]
    assert total == 15.0
