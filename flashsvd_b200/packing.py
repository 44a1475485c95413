"""Device layout of one decoder layer's factors for the decode kernels.

The factors keep the nn.Linear weight layout [out, in] of the reference modules
(utils/model_utils.py:637-643).  Two concatenations are made once at load time so that one rank
projection serves several consumers, as the reference does with its ``packed_qkv_rank`` tensor
(benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:101-127) and its ``PCat`` input
(kernels/mlp/decode/dual_split_triton_pcat_s.py:81-90, up rows first).
"""
from __future__ import annotations

import torch

FACTOR_KEYS = (
    "q_v", "q_u", "k_v", "k_u", "v_v", "v_u", "o_v", "o_u",
    "gate_v", "gate_u", "up_v", "up_u", "down_v", "down_u",
)


def pack_layer(w: dict, *, device, dtype) -> dict:
    """w maps the FACTOR_KEYS plus ``ln1`` / ``ln2`` to weights; returns contiguous device
    tensors named like the fields of ``fsvd_layer`` (without the caches)."""
    def dev(t):
        return t.detach().to(device=device, dtype=dtype).contiguous()

    # q_u, k_u and v_u back to back in one allocation: with equal ranks the kernels then run the
    # three lifts as one stage over the packed matrix (the views below are ordinary row slices)
    q_u, k_u, v_u = w["q_u"], w["k_u"], w["v_u"]
    if q_u.shape[1] == k_u.shape[1] == v_u.shape[1]:
        qkv_u = dev(torch.cat([q_u, k_u, v_u], dim=0))
        nq, nk = q_u.shape[0], k_u.shape[0]
        q_u, k_u, v_u = qkv_u[:nq], qkv_u[nq:nq + nk], qkv_u[nq + nk:]
    else:
        q_u, k_u, v_u = dev(q_u), dev(k_u), dev(v_u)
    return {
        "ln1_w": dev(w["ln1"]),
        "qkv_v": dev(torch.cat([w["q_v"], w["k_v"], w["v_v"]], dim=0)),
        "q_u": q_u,
        "k_u": k_u,
        "v_u": v_u,
        "o_v": dev(w["o_v"]),
        "o_u": dev(w["o_u"]),
        "ln2_w": dev(w["ln2"]),
        "upgate_v": dev(torch.cat([w["up_v"], w["gate_v"]], dim=0)),
        "gate_u": dev(w["gate_u"]),
        "up_u": dev(w["up_u"]),
        "down_v": dev(w["down_v"]),
        "down_u": dev(w["down_u"]),
    }
