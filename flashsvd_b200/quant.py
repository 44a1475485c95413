"""int4-g128 factors for the decode kernels.

The reference stores a quantised linear as ``PackedQuantLinear`` buffers
(src/quant/packed_quant_linear.py:18-35, 126-171): ``qweight uint8 [out, in/2]`` (low nibble =
even input index), ``scales fp16 [out, ceil(in/g)]``, ``zeros int16`` (8 for the symmetric format),
``w = scale * (q - zero)`` with groups along the input dimension (:285-300).  The kernels read a
tiled copy of those buffers (``fsvd_q4_pack`` of the C ABI); nothing is dequantised in HBM.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check

GROUP = 128


@dataclass
class Q4Factor:
    """A [rows, in_features] factor as an int4 tile stream on the device."""

    packed: torch.Tensor          # uint8, the bytes fsvd_q4_pack wrote
    shape: tuple[int, int]
    raw: tuple | None = None      # optional (qweight, scales, zeros) the stream was packed from

    @property
    def is_cuda(self) -> bool:
        return self.packed.is_cuda

    def is_contiguous(self) -> bool:
        return self.packed.is_contiguous()

    def data_ptr(self) -> int:
        return self.packed.data_ptr()

    @property
    def device(self):
        return self.packed.device

    def rows(self, r0: int, r1: int) -> "Q4Factor":
        """View of rows [r0, r1); r0 must be a multiple of 16 (tiles hold 16 rows)."""
        if r0 % 16 or not (0 <= r0 < r1 <= self.shape[0]):
            raise ValueError(f"row slice [{r0}, {r1}) of a {self.shape} int4 factor must start on a multiple of 16")
        K = self.shape[1]
        lib = _lib.load()
        o0 = int(lib.fsvd_q4_packed_bytes(r0, K)) if r0 else 0
        o1 = o0 + int(lib.fsvd_q4_packed_bytes(r1 - r0, K))
        raw = None if self.raw is None else tuple(None if t is None else t[r0:r1] for t in self.raw)
        return Q4Factor(self.packed[o0:o1], (r1 - r0, K), raw)


def pack_int4_codes(q: torch.Tensor) -> torch.Tensor:
    """uint8 codes [out, in] (0..15) -> qweight [out, in/2], low nibble = even input index
    (src/quant/packed_quant_linear.py:18-26)."""
    if q.shape[1] % 2:
        q = torch.cat([q, torch.zeros_like(q[:, :1])], dim=1)
    return (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).contiguous()


def quantize_symmetric(weight: torch.Tensor, group: int = GROUP):
    """(qweight, scales, zeros) of a float weight [out, in], as PackedQuantLinear.pack_weight with
    sym=True produces them (src/quant/packed_quant_linear.py:126-171)."""
    w = weight.detach().to(torch.float32)
    out_f, in_f = w.shape
    ng = (in_f + group - 1) // group
    qs, ss = [], []
    for gi in range(ng):
        chunk = w[:, gi * group:min(in_f, (gi + 1) * group)]
        xmax = torch.maximum(chunk.max(dim=1).values.abs(), chunk.min(dim=1).values.abs())
        xmax = torch.where(xmax == 0, torch.ones_like(xmax), xmax)
        scale = 2.0 * xmax / 15.0
        qs.append(torch.clamp(torch.round(chunk / scale.unsqueeze(1)) + 8.0, 0, 15).to(torch.uint8))
        ss.append(scale.to(torch.float16))
    scales = torch.stack(ss, dim=1).contiguous()
    zeros = torch.full_like(scales, 8, dtype=torch.int16)
    return pack_int4_codes(torch.cat(qs, dim=1)), scales, zeros


def random_q4(out_f: int, in_f: int, *, generator: torch.Generator, device, scale_lo=0.005, scale_hi=0.02,
              group: int = GROUP):
    """Seeded random quantised factor: codes uniform in [-8, 7] (stored + 8), fp16 scales uniform
    in [scale_lo, scale_hi]."""
    ng = (in_f + group - 1) // group
    q = torch.randint(0, 16, (out_f, in_f), device=device, dtype=torch.uint8, generator=generator)
    s = torch.rand(out_f, ng, device=device, generator=generator) * (scale_hi - scale_lo) + scale_lo
    scales = s.to(torch.float16).contiguous()
    return pack_int4_codes(q), scales, torch.full_like(scales, 8, dtype=torch.int16)


def cat_rows(parts):
    """Concatenate (qweight, scales, zeros) triples of equal in_features along the output rows."""
    return tuple(torch.cat([p[i] for p in parts], dim=0).contiguous() for i in range(3))


def pack_q4(qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor | None, in_features: int,
            keep_raw: bool = False) -> Q4Factor:
    """Copy PackedQuantLinear buffers (CUDA tensors) into the tile stream the kernels read.
    ``keep_raw`` keeps references to the source buffers on the factor (for checks against a
    dequantised copy); the kernels never read them."""
    if not (qweight.is_cuda and scales.is_cuda):
        raise ValueError("pack_q4 needs CUDA tensors (there is no CPU path)")
    rows = qweight.shape[0]
    ng = (in_features + GROUP - 1) // GROUP
    if qweight.dtype != torch.uint8 or tuple(qweight.shape) != (rows, in_features // 2):
        raise ValueError(f"qweight must be uint8 [{rows}, {in_features // 2}], got {qweight.dtype} {tuple(qweight.shape)}")
    if scales.dtype != torch.float16 or tuple(scales.shape) != (rows, ng):
        raise ValueError(f"scales must be float16 [{rows}, {ng}], got {scales.dtype} {tuple(scales.shape)}")
    if zeros is not None and (zeros.dtype != torch.int16 or tuple(zeros.shape) != (rows, ng)):
        raise ValueError(f"zeros must be int16 [{rows}, {ng}]")
    lib = _lib.load()
    n = int(lib.fsvd_q4_packed_bytes(rows, in_features))
    out = torch.empty(n, dtype=torch.uint8, device=qweight.device)
    with torch.cuda.device(qweight.device):
        check(lib.fsvd_q4_pack(
            qweight.contiguous().data_ptr(), scales.contiguous().data_ptr(),
            None if zeros is None else zeros.contiguous().data_ptr(), rows, in_features, out.data_ptr(),
            torch.cuda.current_stream().cuda_stream))
    return Q4Factor(out, (rows, in_features), (qweight, scales, zeros) if keep_raw else None)


def pack_layer_q4(q: dict, *, ln1: torch.Tensor, ln2: torch.Tensor, keep_raw: bool = False) -> dict:
    """q maps packing.FACTOR_KEYS to (qweight, scales, zeros, in_features); returns the fields of
    ``fsvd_layer`` (without the caches) with every factor as a Q4Factor.  q_u, k_u and v_u share
    one stream when their ranks agree, so the three lifts run as one stage."""
    def one(key):
        qw, s, z, k = q[key]
        return pack_q4(qw, s, z, k, keep_raw)

    def cat(keys):
        k = q[keys[0]][3]
        if any(q[x][3] != k for x in keys):
            raise ValueError(f"{keys} must share in_features")
        qw, s, z = cat_rows([q[x][:3] for x in keys])
        return pack_q4(qw, s, z, k, keep_raw)

    nq, nk = q["q_u"][0].shape[0], q["k_u"][0].shape[0]
    if q["q_u"][3] == q["k_u"][3] == q["v_u"][3] and nq % 16 == 0 and nk % 16 == 0:
        qkv_u = cat(("q_u", "k_u", "v_u"))
        total = qkv_u.shape[0]
        q_u, k_u, v_u = qkv_u.rows(0, nq), qkv_u.rows(nq, nq + nk), qkv_u.rows(nq + nk, total)
    else:
        q_u, k_u, v_u = one("q_u"), one("k_u"), one("v_u")
    return {
        "ln1_w": ln1, "qkv_v": cat(("q_v", "k_v", "v_v")), "q_u": q_u, "k_u": k_u, "v_u": v_u,
        "o_v": one("o_v"), "o_u": one("o_u"), "ln2_w": ln2, "upgate_v": cat(("up_v", "gate_v")),
        "gate_u": one("gate_u"), "up_u": one("up_u"), "down_v": one("down_v"), "down_u": one("down_u"),
    }
