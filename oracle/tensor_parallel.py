"""CPU restatement of the tensor-parallel layer (test infrastructure, like the rest of oracle/):
one rank's partial sums of a decoder layer on its weight shards, from the building blocks of
``oracle.lowrank_llama``.  ``allreduce`` is any callable that sums a tensor over the ranks."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import lowrank_llama as O


def decode_layer_shard(shape: O.Shape, w: dict, x, k_cache, v_cache, seqlens, cos, sin, *, rank: int, world: int,
                       allreduce):
    """w: the rank's shards (flashsvd_b200.tensor_parallel.shard_layer_weights of the oracle's layer
    dict); k_cache / v_cache [B, S_max, Hk / world, Dh] hold the rank's kv heads."""
    B = x.shape[0]
    Hl, Hkl, Dh = shape.H // world, shape.Hk // world, shape.Dh
    xn = O.rmsnorm(x, w["ln1"], shape.eps)
    q = F.linear(F.linear(xn, w["q_v"]), w["q_u"]).view(B, Hl, Dh)
    k = F.linear(F.linear(xn, w["k_v"]), w["k_u"]).view(B, Hkl, Dh)
    v = F.linear(F.linear(xn, w["v_v"]), w["v_u"]).view(B, Hkl, Dh)
    attn = torch.empty(B, Hl * Dh, dtype=x.dtype)
    for b in range(B):
        pos = int(seqlens[b])
        c, s = cos[pos].unsqueeze(0), sin[pos].unsqueeze(0)
        k_cache[b, pos] = O.rotate_half_apply(k[b], c, s)
        v_cache[b, pos] = v[b]
        attn[b] = O.attend(O.rotate_half_apply(q[b], c, s), k_cache[b, : pos + 1], v_cache[b, : pos + 1]).reshape(-1)
    part = O.lowrank(attn, w["o_v"], w["o_u"])
    h = allreduce(part + x if rank == 0 else part)
    hn = O.rmsnorm(h, w["ln2"], shape.eps)
    act = F.silu(F.linear(F.linear(hn, w["gate_v"]), w["gate_u"])) * F.linear(F.linear(hn, w["up_v"]), w["up_u"])
    part2 = F.linear(F.linear(act, w["down_v"]), w["down_u"])
    return allreduce(part2 + h if rank == 0 else part2)
