"""Tensor-level wrappers over the C ABI.

PyTorch is used for device memory and the current CUDA stream only; every function enqueues one
kernel launch through libflashsvd_b200.so on ``torch.cuda.current_stream()`` and does not
synchronise.  Argument errors raise ``ValueError`` before anything is launched, like the
reference wrappers (kernels/mlp/decode/dual_split_triton_pcat_s.py:139-155).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import FsvdDims, FsvdLayer, LAYER_FIELDS, check


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if dtype == torch.float32:
        return _lib.DTYPE_F32
    raise ValueError(f"flashsvd_b200 supports bfloat16 and float32 tensors, got {dtype}")


def _is_q4(w) -> bool:
    return hasattr(w, "packed")


def _code(x: torch.Tensor, *factors) -> int:
    """dtype code of a call: the activations' type, or DTYPE_BF16_Q4 when the factors are int4
    tile streams (quant.Q4Factor; all of them must be, and the activations bfloat16)."""
    nq = sum(1 for w in factors if w is not None and _is_q4(w))
    if nq == 0:
        return _dtype_code(x.dtype)
    if nq != sum(1 for w in factors if w is not None) or x.dtype != torch.bfloat16:
        raise ValueError("int4 factors need bfloat16 activations and every factor of the call quantised")
    return _lib.DTYPE_BF16_Q4


def _ptr(t) -> int | None:
    if t is None:
        return None
    if _is_q4(t):
        t = t.packed
    if not t.is_cuda:
        raise ValueError("flashsvd_b200 ops need CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("flashsvd_b200 ops need contiguous tensors")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def set_launch_config(warps: int = 0, depth: int = 0, grid: int = 0) -> None:
    """Pick the kernel geometry (see fsvd_set_launch_config in include/flashsvd_b200.h)."""
    check(_lib.load().fsvd_set_launch_config(int(warps), int(depth), int(grid)))


def set_wait_limit(sm_clocks: int) -> None:
    """Budget of every device-side wait in SM clocks (see fsvd_set_wait_limit)."""
    check(_lib.load().fsvd_set_wait_limit(int(sm_clocks)))


def launch_count() -> int:
    return int(_lib.load().fsvd_launch_count())


@dataclass
class Workspace:
    """Scratch for the per-op entry points: rank-space partial sums, the SwiGLU activation,
    attention split partials and the grid-barrier words."""

    buf: torch.Tensor
    nbytes: int

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def status(self) -> int:
        """Blocking read of the device status word; raises if a device-side wait ran out."""
        st = C.c_int(0)
        check(_lib.load().fsvd_workspace_status(self.ptr, C.byref(st)))
        return int(st.value)

    def raw_status(self) -> int:
        """The status word itself (blocking), without the exception."""
        st = C.c_int(0)
        _lib.load().fsvd_workspace_status(self.ptr, C.byref(st))
        return int(st.value)

    def clear_status(self) -> None:
        check(_lib.load().fsvd_workspace_clear_status(self.ptr, _stream()))


def make_dims(*, dtype, B=1, d=8, H=1, Hk=1, Dh=64, I=8, Rq=8, Rk=8, Rv=8, Ro=8, Rg=8, Ru=8,
              Rd=8, S_max=1, vocab=0, n_layers=0, eps=1e-6, rows_are_positions=0) -> FsvdDims:
    """rows_are_positions=1: the B rows are consecutive positions of one sequence (a chunk of its
    prompt) that share cache row 0; cache_seqlens[b] must be first + b."""
    return FsvdDims(_dtype_code(dtype) if isinstance(dtype, torch.dtype) else int(dtype), B, d, H,
                    Hk, Dh, I, Rq, Rk, Rv, Ro, Rg, Ru, Rd, S_max, vocab, n_layers, eps,
                    int(rows_are_positions))


def make_workspace(dims: FsvdDims, device) -> Workspace:
    lib = _lib.load()
    n = int(lib.fsvd_workspace_bytes(C.byref(dims)))
    buf = torch.zeros(n, dtype=torch.uint8, device=device)
    return Workspace(buf, n)


def lowrank_proj(x, v_w, u_w, ws: Workspace, residual=None, out=None):
    """y = (residual +) x @ v_w.T @ u_w.T for x[B, d_in], v_w[R, d_in], u_w[d_out, R]."""
    if x.ndim != 2:
        raise ValueError(f"x must be [B, d_in], got {tuple(x.shape)}")
    B, d_in = x.shape
    if len(v_w.shape) != 2 or v_w.shape[1] != d_in:
        raise ValueError(f"v_w must be [R, {d_in}], got {tuple(v_w.shape)}")
    R = v_w.shape[0]
    if len(u_w.shape) != 2 or u_w.shape[1] != R:
        raise ValueError(f"u_w must be [d_out, {R}], got {tuple(u_w.shape)}")
    d_out = u_w.shape[0]
    if out is None:
        out = torch.empty((B, d_out), dtype=x.dtype, device=x.device)
    check(_lib.load().fsvd_lowrank_proj(
        _ptr(x), _ptr(v_w), _ptr(u_w), _ptr(residual), _ptr(out), B, d_in, R, d_out,
        _code(x, v_w, u_w), ws.ptr, ws.nbytes, _stream()))
    return out


def lift(p, u_w, ws: Workspace, residual=None, out=None):
    """y = (residual +) p @ u_w.T for p[B, R], u_w[d_out, R] (one factor, no rank step)."""
    if p.ndim != 2:
        raise ValueError(f"p must be [B, R], got {tuple(p.shape)}")
    B, R = p.shape
    if len(u_w.shape) != 2 or u_w.shape[1] != R:
        raise ValueError(f"u_w must be [d_out, {R}], got {tuple(u_w.shape)}")
    d_out = u_w.shape[0]
    if out is None:
        out = torch.empty((B, d_out), dtype=p.dtype, device=p.device)
    check(_lib.load().fsvd_lift(_ptr(p), _ptr(u_w), _ptr(residual), _ptr(out), B, R, d_out,
                                _code(p, u_w), ws.ptr, ws.nbytes, _stream()))
    return out


def lowrank_proj_static(x, v_w, u_w, residual=None, out=None):
    """lowrank_proj on the library's built-in scratch (B * R <= 8192): no workspace argument and
    no device allocation inside the call when ``out`` is given.  Calls share one scratch array
    per device and must not overlap in time."""
    if x.ndim != 2:
        raise ValueError(f"x must be [B, d_in], got {tuple(x.shape)}")
    B, d_in = x.shape
    if v_w.ndim != 2 or v_w.shape[1] != d_in:
        raise ValueError(f"v_w must be [R, {d_in}], got {tuple(v_w.shape)}")
    R = v_w.shape[0]
    if u_w.ndim != 2 or u_w.shape[1] != R:
        raise ValueError(f"u_w must be [d_out, {R}], got {tuple(u_w.shape)}")
    d_out = u_w.shape[0]
    if out is None:
        out = torch.empty((B, d_out), dtype=x.dtype, device=x.device)
    check(_lib.load().fsvd_lowrank_proj_static(
        _ptr(x), _ptr(v_w), _ptr(u_w), _ptr(residual), _ptr(out), B, d_in, R, d_out,
        _dtype_code(x.dtype), _stream()))
    return out


def mlp_swiglu_decode(x, gate_u, up_u, down_v, down_u, ws: Workspace, *, upgate_v=None,
                      norm_w=None, eps=1e-6, residual=None, out=None):
    """Fused low-rank SwiGLU MLP for one token per row of x.

    With ``upgate_v`` ([Ru+Rg, d], up rows first) x is the hidden state [B, d]; without it x is
    PCat [B, Ru+Rg] = [p_up | p_gate].  gate_u/up_u are [I, R], down_v [Rd, I], down_u [d, Rd].
    """
    if x.ndim != 2:
        raise ValueError(f"x must be 2-D, got {tuple(x.shape)}")
    B = x.shape[0]
    I, Rg = gate_u.shape
    if tuple(up_u.shape) != tuple(gate_u.shape):
        raise ValueError(f"up_u shape {tuple(up_u.shape)} must match gate_u shape {tuple(gate_u.shape)}")
    Ru = up_u.shape[1]
    if len(down_v.shape) != 2 or down_v.shape[1] != I:
        raise ValueError(f"down_v must be [Rd, {I}], got {tuple(down_v.shape)}")
    Rd = down_v.shape[0]
    if len(down_u.shape) != 2 or down_u.shape[1] != Rd:
        raise ValueError(f"down_u must be [d, {Rd}], got {tuple(down_u.shape)}")
    d = down_u.shape[0]
    if upgate_v is not None:
        if tuple(upgate_v.shape) != (Ru + Rg, d) or x.shape[1] != d:
            raise ValueError(f"upgate_v must be [{Ru + Rg}, {d}] and x [B, {d}]")
    elif x.shape[1] != Ru + Rg:
        raise ValueError(f"PCat must be [B, {Ru + Rg}], got {tuple(x.shape)}")
    if out is None:
        out = torch.empty((B, d), dtype=x.dtype, device=x.device)
    check(_lib.load().fsvd_mlp_swiglu_decode(
        _ptr(x), _ptr(norm_w), float(eps), _ptr(upgate_v), _ptr(gate_u), _ptr(up_u), _ptr(down_v),
        _ptr(down_u), _ptr(residual), _ptr(out), B, d, I, Ru, Rg, Rd,
        _code(x, upgate_v, gate_u, up_u, down_v, down_u), ws.ptr, ws.nbytes, _stream()))
    return out


def qkv_rope_append(x, qkv_v, q_u, k_u, v_u, cos, sin, k_cache, v_cache, cache_seqlens,
                    ws: Workspace, *, num_heads, num_kv_heads, head_dim, ranks, norm_w=None,
                    eps=1e-6, q_out=None):
    """Rank-project, lift, rotate and append the current token; returns the rotated q[B,H,Dh]."""
    B, d = x.shape
    Rq, Rk, Rv = (int(r) for r in ranks)
    if tuple(qkv_v.shape) != (Rq + Rk + Rv, d):
        raise ValueError(f"qkv_v must be [{Rq + Rk + Rv}, {d}], got {tuple(qkv_v.shape)}")
    if tuple(q_u.shape) != (num_heads * head_dim, Rq):
        raise ValueError(f"q_u must be [{num_heads * head_dim}, {Rq}], got {tuple(q_u.shape)}")
    if tuple(k_u.shape) != (num_kv_heads * head_dim, Rk) or tuple(v_u.shape) != (num_kv_heads * head_dim, Rv):
        raise ValueError("k_u / v_u must be [Hk*Dh, Rk] / [Hk*Dh, Rv]")
    if k_cache.ndim != 4 or k_cache.shape[0] < B or tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim):
        raise ValueError(f"k_cache must be [>=B, S, {num_kv_heads}, {head_dim}], got {tuple(k_cache.shape)}")
    if v_cache.shape != k_cache.shape:
        raise ValueError("v_cache shape must match k_cache")
    S_max = k_cache.shape[1]
    if cos.shape[0] < S_max or cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
        raise ValueError(f"cos/sin must be [>={S_max}, {head_dim // 2}]")
    if cache_seqlens.dtype != torch.int32 or cache_seqlens.numel() < B:
        raise ValueError("cache_seqlens must be int32 [B]")
    if k_cache.shape[0] != B and B > 1:
        raise ValueError("k_cache batch dimension must equal B")
    if q_out is None:
        q_out = torch.empty((B, num_heads, head_dim), dtype=x.dtype, device=x.device)
    check(_lib.load().fsvd_qkv_rope_append(
        _ptr(x), _ptr(norm_w), float(eps), _ptr(qkv_v), _ptr(q_u), _ptr(k_u), _ptr(v_u),
        _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), _ptr(cache_seqlens), _ptr(q_out),
        B, d, num_heads, num_kv_heads, head_dim, Rq, Rk, Rv, S_max, _code(x, qkv_v, q_u, k_u, v_u),
        ws.ptr, ws.nbytes, _stream()))
    return q_out


def flash_decode(q, k_cache, v_cache, cache_seqlens, ws: Workspace, *, seqlen_add=0, scale=0.0,
                 out=None):
    """Split-KV single-query attention over cache positions [0, cache_seqlens[b]+seqlen_add)."""
    if q.ndim != 3:
        raise ValueError(f"q must be [B, H, Dh], got {tuple(q.shape)}")
    B, H, Dh = q.shape
    if k_cache.ndim != 4 or k_cache.shape[3] != Dh or v_cache.shape != k_cache.shape:
        raise ValueError("k_cache / v_cache must be [B, S, Hk, Dh]")
    if k_cache.shape[0] != B:
        raise ValueError("cache batch dimension must equal B")
    S_max, Hk = k_cache.shape[1], k_cache.shape[2]
    if cache_seqlens.dtype != torch.int32 or cache_seqlens.numel() < B:
        raise ValueError("cache_seqlens must be int32 [B]")
    if out is None:
        out = torch.empty_like(q)
    check(_lib.load().fsvd_flash_decode(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(cache_seqlens), int(seqlen_add), _ptr(out),
        B, H, Hk, Dh, S_max, float(scale), _dtype_code(q.dtype), ws.ptr, ws.nbytes, _stream()))
    return out


def make_layer_struct(tensors: dict) -> FsvdLayer:
    layer = FsvdLayer()
    for name in LAYER_FIELDS:
        setattr(layer, name, _ptr(tensors[name]))
    return layer


def decode_layer(dims: FsvdDims, layer: FsvdLayer, cos, sin, cache_seqlens, x_in, x_out,
                 ws: Workspace):
    """One decoder layer for one new token per sequence; x_in/x_out are [B, d] in the model dtype."""
    check(_lib.load().fsvd_decode_layer(
        C.byref(dims), C.byref(layer), _ptr(cos), _ptr(sin), _ptr(cache_seqlens), _ptr(x_in),
        _ptr(x_out), ws.ptr, ws.nbytes, _stream()))
    return x_out


def make_tp_workspace(dims: FsvdDims, device) -> Workspace:
    """Workspace of the tensor-parallel layer (tiled path at every batch size)."""
    n = int(_lib.load().fsvd_tp_workspace_bytes(C.byref(dims)))
    if n == 0:
        check(-2)
    return Workspace(torch.zeros(n, dtype=torch.uint8, device=device), n)


def tp_decode_layer(dims: FsvdDims, layer: FsvdLayer, cos, sin, cache_seqlens, x_in, x_out, exchange, ws: Workspace, *,
                    x_norm_in=None, next_norm_w=None, x_norm_out=None):
    """One decoder layer on this rank's shards; the partial sums of the output projection and of the
    down projection are exchanged with the other ranks inside the kernels (``exchange``: the handle of
    a ``tensor_parallel.PeerExchange``).  x_out is the full layer output, the same on every rank.
    ``x_norm_in``: ln1-normalised x_in the caller already holds; ``next_norm_w`` / ``x_norm_out``: also
    write rmsnorm(x_out) * next_norm_w (the next layer's input norm, or the final norm)."""
    check(_lib.load().fsvd_tp_decode_layer(
        C.byref(dims), C.byref(layer), _ptr(cos), _ptr(sin), _ptr(cache_seqlens), _ptr(x_in), _ptr(x_norm_in),
        _ptr(x_out), _ptr(next_norm_w), _ptr(x_norm_out), exchange, ws.ptr, ws.nbytes, _stream()))
    return x_out
