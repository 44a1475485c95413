"""Host-side mirror of the reference's runtime surface for the mode="flashsvd" decode path.

Same names, argument meaning and error behaviour as the reference, so that call sites and tests
written against the reference read the same here:

* ``configure_runtime`` / ``runtime_env_snapshot`` (scripts/demo_support/api.py:20-143),
* ``FlashSVDV15DenseKVCache`` (runtime/cache/attn_dense_kv.py:7-357),
* ``flashsvd_mlp_dual_split_triton_pcat_s`` (kernels/mlp/decode/dual_split_triton_pcat_s.py:123-218),
* ``pack_qkv_shared_bases`` / ``reconstruct_qkv_token_shared_prepacked``
  (kernels/attn/decode/densekv_reconstruct_triton.py:662-760),
* ``generate_text`` (scripts/demo_support/api.py:326-400) on a ``DecodeEngine``.

Device work goes through the C ABI (``ops``); there is no CPU compute path: the kernel wrappers
raise on non-CUDA tensors, as the reference's do.
"""
from __future__ import annotations

import os
from typing import Any, Optional

import torch

# The 15 switches the reference's serving path reads from the environment, in its order.
RUNTIME_ENV_VARS = (
    "SVDLLM_FLASH_FALLBACK",
    "FLASH_SVD_DISABLE_FFN",
    "FLASH_SVD_BASELINE_LR_KVCACHE",
    "FLASH_SVD_ENABLE_DENSE_ATTN_DECODE",
    "FLASH_SVD_DENSE_DECODE_BACKEND",
    "FLASH_SVD_DENSE_DECODE_GRAPH",
    "FLASH_SVD_DENSE_DECODE_AUTOTUNE_SCOPE",
    "FLASH_SVD_USE_CUTLASS_ROPEATTN",
    "FLASH_SVD_BASELINE_DENSE_KVCACHE",
    "FLASH_SVD_REFERENCE_DENSE_ATTN",
    "FLASH_SVD_ENABLE_EXPERIMENTAL_FFN",
    "FLASH_SVD_MLP_CUDA_GRAPH",
    "FLASH_SVD_MLP_CUDA_GRAPH_ALIAS_OUTPUT",
    "FLASH_SVD_MLP_CUDA_GRAPH_SCOPE",
    "FLASH_SVD_FFN_BACKEND",
)

# FFN backends for which the reference also raises FLASH_SVD_ENABLE_EXPERIMENTAL_FFN
# (scripts/demo_support/api.py:54-69).
_EXPERIMENTAL_FFN_BACKENDS = frozenset(
    ["flashsvd_mlp_dual_split_" + s for s in ("prod", "cutlass", "triton_v1", "triton_v2", "triton_v2_sm80", "triton_v3")]
    + ["dual_split_" + s for s in ("cublas", "cutlass", "kernel", "kernel_v2", "kernel_v2_sm80", "kernel_v3")])


def runtime_env_snapshot() -> dict:
    return {name: os.getenv(name) for name in RUNTIME_ENV_VARS}


def _apply_env(settings: dict) -> None:
    """True -> "1", False / None -> unset, anything else -> str(value)."""
    for name, value in settings.items():
        if value is True:
            os.environ[name] = "1"
        elif value is False or value is None:
            os.environ.pop(name, None)
        else:
            os.environ[name] = str(value)


def configure_runtime(mode: str = "flashsvd", *, ffn_backend: str = "auto", enable_mlp_graph: bool = True,
                      mlp_graph_scope: str = "layer_tail", graph_alias_output: bool = False,
                      enable_flash_dense_attn: bool = True, dense_decode_backend: str = "auto",
                      enable_dense_decode_graph: bool = True, dense_decode_autotune_scope: str = "attention",
                      enable_cutlass_rope_attn: bool = False) -> dict:
    """Set the environment switches of the serving path and return their snapshot.

    ``mode="flashsvd"`` selects the dense-KV decode route and the production MLP backend,
    ``"hf"`` / ``"baseline"`` the plain PyTorch path; any other mode is a ValueError.
    """
    key = str(mode).strip().lower().replace("-", "_")
    if key not in ("flashsvd", "hf", "baseline"):
        raise ValueError(f"Unsupported runtime mode: {mode}")
    flash = key == "flashsvd"
    attn = bool(enable_flash_dense_attn) and flash
    backend_key = str(ffn_backend).strip().lower().replace("-", "_")
    _apply_env({
        "SVDLLM_FLASH_FALLBACK": not flash,
        "FLASH_SVD_DISABLE_FFN": not flash,
        "FLASH_SVD_BASELINE_LR_KVCACHE": False,
        "FLASH_SVD_ENABLE_DENSE_ATTN_DECODE": attn,
        "FLASH_SVD_DENSE_DECODE_BACKEND": str(dense_decode_backend) if attn else None,
        "FLASH_SVD_DENSE_DECODE_GRAPH": bool(enable_dense_decode_graph) and attn,
        "FLASH_SVD_DENSE_DECODE_AUTOTUNE_SCOPE": str(dense_decode_autotune_scope) if attn else None,
        "FLASH_SVD_USE_CUTLASS_ROPEATTN": bool(enable_cutlass_rope_attn) and flash,
        "FLASH_SVD_BASELINE_DENSE_KVCACHE": False,
        "FLASH_SVD_REFERENCE_DENSE_ATTN": False,
        "FLASH_SVD_ENABLE_EXPERIMENTAL_FFN": flash and backend_key in _EXPERIMENTAL_FFN_BACKENDS,
        "FLASH_SVD_MLP_CUDA_GRAPH": bool(enable_mlp_graph) and flash,
        "FLASH_SVD_MLP_CUDA_GRAPH_ALIAS_OUTPUT": bool(graph_alias_output) and flash,
        "FLASH_SVD_MLP_CUDA_GRAPH_SCOPE": str(mlp_graph_scope) if flash else None,
        "FLASH_SVD_FFN_BACKEND": str(ffn_backend) if flash else None,
    })
    return runtime_env_snapshot()


# --------------------------------------------------------------------------------- KV cache
try:   # the reference's cache is a transformers Cache (runtime/cache/attn_dense_kv.py:4-7)
    from transformers.cache_utils import Cache as _CacheBase
except Exception:   # pragma: no cover - transformers is optional for the kernel-level API
    class _CacheBase:   # type: ignore
        def __init__(self, *a, **k):
            pass


class FlashSVDV15DenseKVCache(_CacheBase):
    """Dense KV cache in the layout the decode kernels read: ``key_cache[l]`` / ``value_cache[l]``
    are ``[max_batch, max_cache_len, Hk, Dh]``, zero-initialised, shaped on first use; K is stored
    after RoPE; the number of tokens seen is advanced by layer 0 only."""

    is_compileable = False

    def __init__(self, config, *, max_batch_size: int, max_cache_len: int, device=None,
                 dtype: torch.dtype = torch.float16, layer_device_map: Optional[dict] = None) -> None:
        try:   # transformers 5.x wants the layer list, 4.x takes no argument (attn_dense_kv.py:29-32)
            super().__init__(layers=[])
        except TypeError:
            super().__init__()
        self._config = config
        self._max_batch_size = int(max_batch_size)
        self._max_cache_len = int(max_cache_len)
        self._dtype = dtype
        self._rope_theta = float(getattr(config, "rope_theta", 10000.0))
        self._seen_tokens = 0
        self.key_cache: list = []
        self.value_cache: list = []
        self._layer_initialized: list = []
        self._layer_device: list = []
        self._fa2_cache_seqlens: dict = {}
        self._rope_cache: dict = {}
        for idx in range(int(getattr(config, "num_hidden_layers", 0))):
            if layer_device_map is not None:
                d = layer_device_map[idx]
                d = torch.device("cuda", d) if isinstance(d, int) else torch.device(d)
            else:
                d = torch.device(device) if device is not None else torch.device("cpu")
            self._layer_device.append(d)
            empty = torch.zeros((self._max_batch_size, self._max_cache_len, 0, 0), dtype=dtype, device=d)
            self.key_cache.append(empty)
            self.value_cache.append(empty.clone())
            self._layer_initialized.append(False)

    @property
    def max_batch_size(self) -> int:
        return self._max_batch_size

    @property
    def max_cache_len(self) -> int:
        return self._max_cache_len

    def __len__(self) -> int:
        return len(self.key_cache)

    def _ensure_layer_spec(self, layer_idx: int, *, h: int, dh: int) -> None:
        kc = self.key_cache[layer_idx]
        if (int(kc.shape[2]), int(kc.shape[3])) == (int(h), int(dh)):
            return
        if self._layer_initialized[layer_idx]:
            raise RuntimeError(
                f"FlashSVDV15DenseKVCache shape changed after init for layer {layer_idx}: "
                f"old={(int(kc.shape[2]), int(kc.shape[3]))}, new={(int(h), int(dh))}")
        shape = (self._max_batch_size, self._max_cache_len, int(h), int(dh))
        self.key_cache[layer_idx] = torch.zeros(shape, dtype=self._dtype, device=self._layer_device[layer_idx])
        self.value_cache[layer_idx] = torch.zeros_like(self.key_cache[layer_idx])

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict] = None):
        """Prefill / baseline write: key_states, value_states are [B, Hk, L, Dh] (K after RoPE),
        written at ``cache_kwargs["cache_position"]`` (default: appended); returns the valid
        prefix as [B, Hk, S, Dh] like a transformers cache."""
        layer_idx = int(layer_idx)
        B, Hk, L, Dh = (int(v) for v in key_states.shape)
        self._ensure_layer_spec(layer_idx, h=Hk, dh=Dh)
        self._layer_initialized[layer_idx] = True
        if B > self._max_batch_size:
            raise RuntimeError(f"batch {B} exceeds max_batch_size {self._max_batch_size}")
        pos = None if cache_kwargs is None else cache_kwargs.get("cache_position")
        if pos is None:
            pos = torch.arange(self._seen_tokens, self._seen_tokens + L, device=key_states.device)
        pos = pos.to(device=self.key_cache[layer_idx].device, dtype=torch.long).reshape(-1)
        if int(pos.numel()) != L:
            raise ValueError(f"cache_position has {int(pos.numel())} entries for {L} new tokens")
        end = int(pos.max().item()) + 1 if L else self._seen_tokens
        if end > self._max_cache_len:
            raise IndexError(f"cache position {end - 1} outside max_cache_len {self._max_cache_len}")
        self.key_cache[layer_idx][:B].index_copy_(1, pos, key_states.transpose(1, 2).to(self._dtype))
        self.value_cache[layer_idx][:B].index_copy_(1, pos, value_states.transpose(1, 2).to(self._dtype))
        if layer_idx == 0:
            self._seen_tokens = max(self._seen_tokens, end)
        k = self.key_cache[layer_idx][:B, :end].transpose(1, 2)
        v = self.value_cache[layer_idx][:B, :end].transpose(1, 2)
        return k, v

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return int(self._seen_tokens)

    def get_max_cache_shape(self) -> Optional[int]:
        return self._max_cache_len

    def get_mask_sizes(self, cache_position, layer_idx: int = 0):
        q_len = int(cache_position.shape[0]) if torch.is_tensor(cache_position) else int(cache_position)
        return q_len + self.get_seq_length(), 0

    def _seqlens_buffer(self, layer_idx: int, batch_size: int) -> torch.Tensor:
        key = (int(layer_idx), int(batch_size))
        dev = self.key_cache[layer_idx].device
        buf = self._fa2_cache_seqlens.get(key)
        if buf is None or buf.device != dev:
            buf = torch.empty((int(batch_size),), device=dev, dtype=torch.int32)
            self._fa2_cache_seqlens[key] = buf
        return buf

    def prepare_fa2_step(self, layer_idx: int, *, batch_size: int, cache_position=None):
        """(k_cache[:B], v_cache[:B], cache_seqlens int32[B]) for one decode step: the write
        position is ``cache_position`` when given (scalar, 1 entry or one per row), else the
        number of tokens seen."""
        layer_idx = int(layer_idx)
        B = int(batch_size)
        sl = self._seqlens_buffer(layer_idx, B)
        if cache_position is None:
            sl.fill_(self._seen_tokens)
        elif torch.is_tensor(cache_position):
            pos = cache_position.to(device=sl.device, dtype=torch.int32).reshape(-1)
            if int(pos.numel()) == 0:
                sl.zero_()
            elif int(pos.numel()) == 1:
                sl.copy_(pos.expand_as(sl))
            else:
                sl.copy_(pos[:B])
        else:
            sl.fill_(int(cache_position))
        return self.key_cache[layer_idx][:B], self.value_cache[layer_idx][:B], sl

    def prepare_fa2_direct_write_step(self, layer_idx: int, *, batch_size: int, num_heads: int, head_dim: int,
                                      q_len: int, cache_position=None):
        """(k_cache[:B], v_cache[:B], k_slot, v_slot, cache_seqlens) for a step whose new key / value
        are written by the caller straight into ``k_slot`` / ``v_slot`` = cache[:, start:start + 1];
        ``cache_seqlens`` is filled with start + 1 (the keys to attend).  None when q_len != 1 or the
        positions differ per row; IndexError past the end (runtime/cache/attn_dense_kv.py:258-311)."""
        layer_idx, B, q_len = int(layer_idx), int(batch_size), int(q_len)
        if q_len != 1:
            return None
        self._ensure_layer_spec(layer_idx, h=int(num_heads), dh=int(head_dim))
        kc_full, vc_full = self.key_cache[layer_idx], self.value_cache[layer_idx]
        if cache_position is None:
            start = int(self.get_seq_length())
        elif torch.is_tensor(cache_position):
            pos = cache_position.to(dtype=torch.int64).reshape(-1)
            if int(pos.numel()) == 0:
                return None
            first = int(pos[0].item())
            if int(pos.numel()) > 1 and bool(torch.any(pos != first).item()):
                return None
            start = first
        else:
            start = int(cache_position)
        if start < 0 or start + q_len > self._max_cache_len:
            raise IndexError(f"FlashSVDV15DenseKVCache write position out of range: start={start} q_len={q_len} "
                             f"max={self._max_cache_len}")
        kc, vc = kc_full[:B], vc_full[:B]
        sl = self._seqlens_buffer(layer_idx, B)
        sl.fill_(start + q_len)
        self._layer_initialized[layer_idx] = True
        return kc, vc, kc[:, start:start + q_len], vc[:, start:start + q_len], sl

    def get_fa2_kvcache(self, layer_idx: int, *, batch_size: int):
        return self.prepare_fa2_step(layer_idx, batch_size=batch_size, cache_position=None)

    def advance_after_fa2(self, layer_idx: int, *, q_len: int, cache_position=None) -> None:
        if int(layer_idx) != 0:
            return
        on_host = cache_position is not None and torch.is_tensor(cache_position) and not cache_position.is_cuda
        if on_host and int(cache_position.numel()) > 0:
            self._seen_tokens = max(self._seen_tokens, int(cache_position.max().item()) + 1)
        else:
            self._seen_tokens = self._seen_tokens + int(q_len)

    def get_rope_tables(self, seqlen: int, head_dim: int, *, device, dtype: torch.dtype):
        """cos, sin [seqlen, head_dim/2]: fp32 angles pos * theta^(-i/half), cast to ``dtype``."""
        key = (int(seqlen), int(head_dim), str(device), dtype)
        hit = self._rope_cache.get(key)
        if hit is not None:
            return hit
        half = int(head_dim) // 2
        pos = torch.arange(int(seqlen), device=device, dtype=torch.float32)
        inv_freq = 1.0 / (self._rope_theta ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
        ang = torch.einsum("m,d->md", pos, inv_freq)
        out = (torch.cos(ang).to(dtype).contiguous(), torch.sin(ang).to(dtype).contiguous())
        self._rope_cache[key] = out
        return out


class FlashSVDLegacySparseKVCache:
    """Name of the reference's rank-space cache (runtime/cache/attn_legacy_sparse_kv.py:23-257: it
    keeps x . k_v^T and x . v_v^T per position and rebuilds keys and values inside its own decode
    kernels).  That is another decode mode than the dense-cache path this package serves; the name
    is importable, constructing it says so."""

    def __init__(self, *args, **kwargs):
        raise NotImplementedError("the rank-space KV cache belongs to the reference's legacy decode mode; flashsvd_b200 "
                                  "serves mode='flashsvd' with FlashSVDV15DenseKVCache")


LowRankKVCache = FlashSVDLegacySparseKVCache   # the reference's alias (runtime/cache/attn_legacy_sparse_kv.py:260)


# --------------------------------------------------------------------------------- kernel wrappers
_layout_cache: dict = {}
_workspaces: dict = {}


def _as_linear_weight(t: torch.Tensor) -> torch.Tensor:
    """The reference passes factors transposed ([in, out] = weight.t().contiguous()); the kernels
    read the nn.Linear layout [out, in].  The transposed copy is made once per tensor object: an
    entry is valid only while the very tensor it was made from is alive and unmodified (a new
    tensor may reuse a freed tensor's address)."""
    import weakref

    key = (t.data_ptr(), tuple(t.shape), t.dtype)
    hit = _layout_cache.get(key)
    if hit is not None and hit[0]() is t and hit[1] == t._version:
        return hit[2]
    if len(_layout_cache) > 512:
        _layout_cache.clear()
    out = t.t().contiguous()
    _layout_cache[key] = (weakref.ref(t), t._version, out)
    return out


def _workspace(device, dtype, B: int, **sizes):
    from . import ops

    key = (str(device), dtype, int(B), tuple(sorted(sizes.items())))
    ws = _workspaces.get(key)
    if ws is None:
        ws = ops.make_workspace(ops.make_dims(dtype=dtype, B=B, **sizes), device)
        _workspaces[key] = ws
    return ws


def flashsvd_mlp_dual_split_triton_pcat_s(PCat, GateU, UpU, DownV, DownU, b2=None, *, BT=None, BR=None, BD=None,
                                          BR2=None, num_warps=None, num_stages=None, workspace_s2d=None):
    """y[B, L, H] = (silu(p_gate @ GateU) * (p_up @ UpU)) @ DownV @ DownU (+ b2) for PCat =
    [p_up | p_gate] of one token per sequence.  The tile-size arguments of the reference are
    accepted and ignored; ``workspace_s2d`` is not needed."""
    assert PCat.is_cuda and GateU.is_cuda and UpU.is_cuda and DownV.is_cuda and DownU.is_cuda
    if PCat.ndim != 3:
        raise ValueError(f"PCat must be [B, L, 2R], got {tuple(PCat.shape)}")
    B, L, two_r = (int(v) for v in PCat.shape)
    if two_r % 2 != 0:
        raise ValueError(f"PCat last dim must be even, got {two_r}")
    R = two_r // 2
    if GateU.shape[0] != R:
        raise ValueError(f"GateU must be [R, D] with R={R}, got {tuple(GateU.shape)}")
    if UpU.shape != GateU.shape:
        raise ValueError(f"UpU shape {tuple(UpU.shape)} must match GateU shape {tuple(GateU.shape)}")
    D = int(GateU.shape[1])
    if tuple(DownV.shape) != (D, R):
        raise ValueError(f"DownV must be [D, R]=[{D}, {R}], got {tuple(DownV.shape)}")
    if DownU.ndim != 2 or DownU.shape[0] != R:
        raise ValueError(f"DownU must be [R, H] with R={R}, got {tuple(DownU.shape)}")
    from . import ops

    T = B * L
    Hd = int(DownU.shape[1])
    ws = _workspace(PCat.device, PCat.dtype, T, d=Hd, I=D, Ru=R, Rg=R, Rd=R)
    y = ops.mlp_swiglu_decode(PCat.reshape(T, two_r).contiguous(), _as_linear_weight(GateU), _as_linear_weight(UpU),
                              _as_linear_weight(DownV), _as_linear_weight(DownU), ws)
    if b2 is not None:
        y = y + b2.to(y.dtype)
    return y.reshape(B, L, Hd)


def flashsvd_mlp_dual_split_triton_v1(PUp, PGate, GateU, UpU, DownV, DownU, b2=None, *, BR=None, BD=None, BR2=None,
                                      num_warps=None, num_stages=None, store_partials_fp32: bool = False,
                                      workspace_s2d=None):
    """The split-input form of the decode MLP (kernels/mlp/decode/dual_split_triton.py:535-624 and its
    v2 / v2_sm80 / v3 variants, which differ in tiling and scratch only): PUp and PGate [B, L, R]
    instead of one PCat.  Same arithmetic as ``flashsvd_mlp_dual_split_triton_pcat_s``; the tile
    arguments, ``store_partials_fp32`` and ``workspace_s2d`` are accepted and ignored."""
    assert PUp.is_cuda and PGate.is_cuda and GateU.is_cuda and UpU.is_cuda and DownV.is_cuda and DownU.is_cuda
    if PUp.ndim != 3 or PGate.ndim != 3:
        raise ValueError(f"PUp/PGate must be [B, L, R], got {tuple(PUp.shape)} and {tuple(PGate.shape)}")
    if PUp.shape != PGate.shape:
        raise ValueError(f"PUp and PGate shapes must match, got {tuple(PUp.shape)} and {tuple(PGate.shape)}")
    return flashsvd_mlp_dual_split_triton_pcat_s(torch.cat([PUp, PGate], dim=-1), GateU, UpU, DownV, DownU, b2)


flashsvd_mlp_dual_split_triton_v2 = flashsvd_mlp_dual_split_triton_v1
flashsvd_mlp_dual_split_triton_v2_sm80 = flashsvd_mlp_dual_split_triton_v1
flashsvd_mlp_dual_split_triton_v3 = flashsvd_mlp_dual_split_triton_v1
# the names the reference exports beside them (kernels/mlp/decode/dual_split_triton.py:969-983)
flashsvd_ffn_dual_split_token = flashsvd_mlp_dual_split_triton_v1
flashsvd_ffn_dual_split_token_v2 = flashsvd_mlp_dual_split_triton_v2
flashsvd_ffn_dual_split_token_v2_sm80 = flashsvd_mlp_dual_split_triton_v2_sm80
flashsvd_ffn_dual_split_token_v3 = flashsvd_mlp_dual_split_triton_v3


def pack_qkv_shared_bases(Vq, Vk, Vv):
    """[H|Hk, R, Dh] decode bases -> [R, H*Dh] / [R, Hk*Dh] (rank-major), as the reference packs them."""
    if not (Vq.is_cuda and Vk.is_cuda and Vv.is_cuda):
        raise ValueError("pack_qkv_shared_bases expects CUDA tensors.")
    if Vq.ndim != 3 or Vk.ndim != 3 or Vv.ndim != 3:
        raise ValueError(f"Expected Vq/Vk/Vv to be 3D [H|Hk,R,Dh], got {tuple(Vq.shape)}/{tuple(Vk.shape)}/{tuple(Vv.shape)}")
    Dh = int(Vq.shape[2])
    if Vk.shape[2] != Dh or Vv.shape[2] != Dh:
        raise ValueError("All bases must share the same head_dim.")
    return tuple(v.permute(1, 0, 2).reshape(int(v.shape[1]), int(v.shape[0]) * Dh).contiguous() for v in (Vq, Vk, Vv))


def reconstruct_qkv_token_shared_prepacked(Pq, Pk, Pv, Vq_flat, Vk_flat, Vv_flat, *, H: int, Hk: int, Dh: int,
                                           bq=None, bk=None, bv=None):
    """Q[B,H,Dh], K[B,Hk,Dh], V[B,Hk,Dh] = P* @ V*_flat (+ bias) for the current token."""
    tensors = (Pq, Pk, Pv, Vq_flat, Vk_flat, Vv_flat)
    if not all(t.is_cuda for t in tensors):
        raise ValueError("reconstruct_qkv_token_shared_prepacked expects all tensors on CUDA.")
    if Pq.ndim != 2 or Pk.ndim != 2 or Pv.ndim != 2:
        raise ValueError(f"Expected shared Pq/Pk/Pv to be 2D [B,R], got {tuple(Pq.shape)}/{tuple(Pk.shape)}/{tuple(Pv.shape)}")
    for name, p, v, heads in (("q", Pq, Vq_flat, H), ("k", Pk, Vk_flat, Hk), ("v", Pv, Vv_flat, Hk)):
        if v.ndim != 2 or tuple(v.shape) != (int(p.shape[1]), int(heads) * int(Dh)):
            raise ValueError(f"V{name}_flat must be [{int(p.shape[1])}, {int(heads) * int(Dh)}], got {tuple(v.shape)}")
    from . import ops

    B = int(Pq.shape[0])
    ws = _workspace(Pq.device, Pq.dtype, B)
    outs = []
    for p, v, bias, heads in ((Pq, Vq_flat, bq, H), (Pk, Vk_flat, bk, Hk), (Pv, Vv_flat, bv, Hk)):
        y = ops.lift(p.contiguous(), _as_linear_weight(v), ws)
        if bias is not None:
            y = y + bias.to(y.dtype)
        outs.append(y.reshape(B, int(heads), int(Dh)))
    return tuple(outs)


_head_base_cache: dict = {}


def _lift_heads(P, V, ws):
    """P[B, R] x V[Hx, R, Dh] (per-head bases as the reference modules expose them) -> [B, Hx, Dh].
    The kernels read the nn.Linear layout [Hx * Dh, R]; that copy is made once per base tensor."""
    from . import ops

    Hx, R, Dh = V.shape
    key = (V.data_ptr(), V._version, tuple(V.shape), V.dtype, str(V.device))
    w = _head_base_cache.get(key)
    if w is None:
        if len(_head_base_cache) > 256:
            _head_base_cache.clear()
        w = V.permute(0, 2, 1).reshape(Hx * Dh, R).contiguous()
        _head_base_cache[key] = w
    return ops.lift(P.contiguous(), w, ws).view(P.shape[0], Hx, Dh)


def reconstruct_qkv_token_shared_hetero(Pq, Pk, Pv, Vq, Vk, Vv, *, bq=None, bk=None, bv=None, BD: int = 64,
                                        BR: int = 64, num_warps: int = 4, num_stages: int = 2):
    """Current-token q/k/v from rank space with per-head bases Vq[H, Rq, Dh], Vk[Hk, Rk, Dh],
    Vv[Hk, Rv, Dh] and possibly different ranks; the tile arguments of the reference's Triton
    launch are accepted and ignored (kernels/attn/decode/densekv_reconstruct_triton.py:559-659)."""
    if not all(t.is_cuda for t in (Pq, Pk, Pv, Vq, Vk, Vv)):
        raise ValueError("reconstruct_qkv_token_shared_hetero expects all tensors on CUDA.")
    if Pq.ndim != 2 or Pk.ndim != 2 or Pv.ndim != 2:
        raise ValueError(f"Expected Pq/Pk/Pv to be 2D [B,R*], got {tuple(Pq.shape)}/{tuple(Pk.shape)}/{tuple(Pv.shape)}")
    if Vq.ndim != 3 or Vk.ndim != 3 or Vv.ndim != 3:
        raise ValueError(f"Expected Vq/Vk/Vv to be 3D [H|Hk,R*,Dh], got {tuple(Vq.shape)}/{tuple(Vk.shape)}/{tuple(Vv.shape)}")
    B = Pq.shape[0]
    if Pk.shape[0] != B or Pv.shape[0] != B:
        raise ValueError("Pq/Pk/Pv batch mismatch")
    for P, V, n in ((Pq, Vq, "q"), (Pk, Vk, "k"), (Pv, Vv, "v")):
        if P.shape[1] != V.shape[1]:
            raise ValueError(f"rank mismatch for {n}: P has {P.shape[1]}, V has {V.shape[1]}")
    ws = _workspace(Pq.device, Pq.dtype, B, Ro=max(Pq.shape[1], Pk.shape[1], Pv.shape[1]),
                    d=max(Vq.shape[0] * Vq.shape[2], 8))
    q, k, v = _lift_heads(Pq, Vq, ws), _lift_heads(Pk, Vk, ws), _lift_heads(Pv, Vv, ws)
    if bq is not None:
        q = q + bq.view(1, *q.shape[1:])
    if bk is not None:
        k = k + bk.view(1, *k.shape[1:])
    if bv is not None:
        v = v + bv.view(1, *v.shape[1:])
    return q, k, v


def reconstruct_qkv_token_shared(Pq, Pk, Pv, Vq, Vk, Vv, **kw):
    """The equal-rank form of the same reconstruction (densekv_reconstruct_triton.py:464-556)."""
    if Pq.ndim == 2 and Pk.ndim == 2 and Pv.ndim == 2 and not (Pq.shape[1] == Pk.shape[1] == Pv.shape[1]):
        raise ValueError("reconstruct_qkv_token_shared expects one shared rank; use the _hetero variant")
    return reconstruct_qkv_token_shared_hetero(Pq, Pk, Pv, Vq, Vk, Vv, **kw)


def reconstruct_qkv_token(Pq, Pk, Pv, Vq, Vk, Vv, **kw):
    return reconstruct_qkv_token_shared_hetero(Pq, Pk, Pv, Vq, Vk, Vv, **kw)


def call_flash_attn_with_kvcache(flash_attn_with_kvcache, q_bmhd, k_cache_bmhd, v_cache_bmhd, *, k_bmhd=None,
                                 v_bmhd=None, cache_seqlens=None, rotary_cos=None, rotary_sin=None, causal: bool = True):
    """The reference's call into flash-attn (runtime/attn/decode_registry.py:177-211) served by this
    library: q[B,1,H,Dh] (and the new k / v [B,1,Hk,Dh]) are rotated at position cache_seqlens[b]
    when tables are given, k / v are appended to the caches, and attention runs over
    cache_seqlens[b] + 1 keys (cache_seqlens[b] keys when no new k / v is passed).  The first
    argument (the library function the reference would call) is accepted and not used."""
    del flash_attn_with_kvcache, causal
    if not (q_bmhd.is_cuda and k_cache_bmhd.is_cuda and v_cache_bmhd.is_cuda):
        raise ValueError("call_flash_attn_with_kvcache expects CUDA tensors")
    B, L, H, Dh = q_bmhd.shape
    if L != 1:
        raise ValueError("decode path: one query token per sequence")
    Hk, S_max = k_cache_bmhd.shape[2], k_cache_bmhd.shape[1]
    if cache_seqlens is None:
        raise ValueError("cache_seqlens is required")
    sl = cache_seqlens.to(torch.int32)
    q, k = q_bmhd[:, 0], None if k_bmhd is None else k_bmhd[:, 0]
    if rotary_cos is not None:
        pos = sl.long().clamp_max(rotary_cos.shape[0] - 1)
        cos, sin = rotary_cos[pos][:, None, :].to(q.dtype), rotary_sin[pos][:, None, :].to(q.dtype)
        half = Dh // 2

        def rot(x):
            x1, x2 = x[..., :half], x[..., half:]
            return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

        q = rot(q)
        k = None if k is None else rot(k)
    add = 0
    if k is not None:
        if bool((sl >= S_max).any().item()):
            raise IndexError("cache position outside the cache")
        rows = torch.arange(B, device=q.device)
        k_cache_bmhd[rows, sl.long()] = k.to(k_cache_bmhd.dtype)
        v_cache_bmhd[rows, sl.long()] = v_bmhd[:, 0].to(v_cache_bmhd.dtype)
        add = 1
    from . import ops

    ws = _workspace(q.device, q.dtype, B, H=H, Hk=Hk, Dh=Dh, S_max=S_max)
    out = ops.flash_decode(q.contiguous(), k_cache_bmhd, v_cache_bmhd, sl.contiguous(), ws, seqlen_add=add)
    return out.view(B, 1, H, Dh)


# ---- the other names of runtime/attn/__init__.py:19-33
def maybe_kwargs(fn, kwargs: dict) -> dict:
    """The entries of ``kwargs`` that ``fn`` takes (all of them when its signature cannot be read;
    runtime/attn/decode_registry.py:30-35)."""
    import inspect

    try:
        params = inspect.signature(fn).parameters
    except Exception:
        return kwargs
    return {k: v for k, v in kwargs.items() if k in params}


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None, cache_seqlens=None,
                            causal: bool = True, rotary_interleaved: bool = False, softmax_scale=None, dropout_p: float = 0.0,
                            window_size=(-1, -1), **unsupported):
    """The part of flash-attn's ``flash_attn_with_kvcache`` signature that the reference's decode uses
    (runtime/attn/decode_registry.py:177-211), served by this library."""
    if rotary_interleaved or dropout_p or tuple(window_size) != (-1, -1) or softmax_scale is not None or unsupported:
        raise ValueError("only the decode call of the reference is served: non-interleaved rotary, no dropout, no window, "
                         "default scale")
    return call_flash_attn_with_kvcache(None, q, k_cache, v_cache, k_bmhd=k, v_bmhd=v, cache_seqlens=cache_seqlens,
                                        rotary_cos=rotary_cos, rotary_sin=rotary_sin, causal=causal)


def get_flash_attn_with_kvcache():
    """The reference resolves flash-attn's function here (None when the wheel is missing,
    runtime/attn/decode_registry.py:154-175); this package returns its own implementation."""
    return flash_attn_with_kvcache


def get_flashsvd_v15_attn_densekv_decode_mod():
    """The module that holds ``reconstruct_qkv_token*`` and ``pack_qkv_shared_bases``
    (runtime/attn/decode_registry.py:212-236): here, this module."""
    import sys

    return sys.modules[__name__]


get_dense_token_decode_mod = get_flashsvd_v15_attn_densekv_decode_mod


def _no_legacy_kernels(*_args, **_kwargs):
    raise ImportError("Failed to load any decode attention module: the rank-space (legacy sparse-KV) decode kernels are "
                      "not part of flashsvd_b200, which serves the dense-cache path (mode='flashsvd')")


# the rank-space cache path of the reference (runtime/attn/decode_registry.py:51-150, 238-330) is a different decode
# mode: its registry functions exist and fail the way the reference fails when those kernel files are absent
get_flashsvd_attn_legacy_sparsekv_decode_mods = _no_legacy_kernels
get_flashsvd_decode_attn_mods = _no_legacy_kernels
get_default_flashsvd_attn_legacy_sparsekv_decode_mod = _no_legacy_kernels
get_default_flashsvd_decode_attn_mod = _no_legacy_kernels
resolve_legacy_sparsekv_decode_variant = _no_legacy_kernels
resolve_decode_variant = _no_legacy_kernels
select_legacy_sparsekv_decode_variant = _no_legacy_kernels
select_decode_variant = _no_legacy_kernels


def manual_llama_decode_step(model, input_ids: torch.Tensor, *, past_key_values, cache_position: torch.Tensor,
                             attention_mask=None):
    """One token through embed -> decoder layers -> norm -> lm_head(last), layer by layer, as the
    reference's ``_manual_llama_decode_step`` drives a transformers Llama (utils/evaluator.py:39-82).
    The layers are transformers ``LlamaDecoderLayer``s whose ``self_attn`` / ``mlp`` are this
    package's modules; the decode arithmetic of every layer runs in the CUDA library."""
    from types import SimpleNamespace

    inner = model.model
    hidden_states = inner.embed_tokens(input_ids)
    position_ids = cache_position.unsqueeze(0)
    # the attention modules of this package rotate with the cache's own tables at cache_position, so
    # the transformers rotary embedding is not evaluated (the reference computes it here and its
    # FlashSVD attention ignores it as well)
    position_embeddings = None
    for decoder_layer in inner.layers[: model.config.num_hidden_layers]:
        out = decoder_layer(hidden_states, attention_mask=None, position_ids=position_ids,
                            past_key_values=past_key_values, cache_position=cache_position,
                            position_embeddings=position_embeddings)
        hidden_states = out[0] if isinstance(out, (tuple, list)) else out
    hidden_states = inner.norm(hidden_states)
    logits = model.lm_head(hidden_states[:, -1:, :])
    return SimpleNamespace(logits=logits, past_key_values=past_key_values)


# --------------------------------------------------------------------------------- generation
def _sample_next_token(logits: torch.Tensor, *, do_sample: bool, temperature: float, top_p: float) -> torch.Tensor:
    """Next token ids [B, 1] from logits [B, vocab] as the reference draws them
    (scripts/demo_support/api.py:192-209): argmax unless sampling with a positive temperature; else
    softmax(logits / temperature), and for top_p < 1 the nucleus = the most probable tokens up to and
    including the first one that carries the cumulative probability past top_p, renormalised."""
    if not do_sample or temperature <= 0.0:
        return logits.argmax(dim=-1, keepdim=True)
    probs = torch.softmax(logits / float(max(temperature, 1e-5)), dim=-1)
    if float(top_p) >= 1.0:
        return torch.multinomial(probs, num_samples=1)
    sp, si = torch.sort(probs, dim=-1, descending=True)
    before = torch.cumsum(sp, dim=-1) > float(top_p)        # True where the mass up to and including the token exceeds top_p
    drop = torch.zeros_like(before)
    drop[..., 1:] = before[..., :-1]                         # a token goes when the mass BEFORE it already exceeded top_p
    sp = sp.masked_fill(drop, 0.0)
    sp = sp / sp.sum(dim=-1, keepdim=True).clamp_min(1e-12)
    return torch.gather(si, dim=-1, index=torch.multinomial(sp, num_samples=1))


@torch.inference_mode()
def generate_text(model: Any, tokenizer: Any, *, prompt: str, max_new_tokens: int = 64, device=None,
                  do_sample: bool = False, temperature: float = 0.8, top_p: float = 0.95) -> dict:
    """Single-prompt generation (greedy, or sampled with temperature / top_p) on a ``DecodeEngine``; returns the reference's result dict
    (prompt_token_count, generated_token_count, output_ids, completion_ids, text, completion_text).
    Generation stops after an end-of-sequence token, like the reference loop."""
    from .engine import DecodeEngine, engine_for_model, has_lowrank_modules

    if not isinstance(model, DecodeEngine):
        if not has_lowrank_modules(model):
            if not callable(model) or not hasattr(model, "parameters"):
                raise TypeError("generate_text takes a DecodeEngine, a model with low-rank modules or a transformers model")
            return _generate_text_generic(model, tokenizer, prompt=prompt, max_new_tokens=max_new_tokens, device=device,
                                          do_sample=do_sample, temperature=temperature, top_p=top_p)
        enc0 = tokenizer(prompt, return_tensors="pt", add_special_tokens=False)
        need = int(enc0["input_ids"].shape[1]) + int(max_new_tokens)
        model = engine_for_model(model, batch_size=1, max_cache_len=need + 4)
    enc = tokenizer(prompt, return_tensors="pt", add_special_tokens=False)
    input_ids = enc["input_ids"]
    if int(input_ids.shape[0]) != 1:
        raise ValueError("generate_text currently supports batch_size=1 only.")
    prompt_len = int(input_ids.shape[1])
    max_new_tokens = int(max_new_tokens)
    if prompt_len + max_new_tokens > model.S_max:
        raise IndexError(f"prompt of {prompt_len} tokens + {max_new_tokens} new tokens exceeds the cache length {model.S_max}")
    model.reset()
    model.prefill(input_ids)
    eos = getattr(tokenizer, "eos_token_id", None)
    if do_sample and float(temperature) > 0.0 and max_new_tokens:
        # sampled: the kernel leaves the logits of every step on the device; the token drawn from them
        # on the host side of the API is written back as the next step's input (the kernel's own greedy
        # choice is overwritten), one launch per token
        new = []
        for i in range(max_new_tokens):
            nxt = _sample_next_token(model.logits[:1].float(), do_sample=True, temperature=temperature, top_p=top_p)
            new.append(int(nxt[0, 0]))
            if (eos is not None and new[-1] == int(eos)) or i + 1 == max_new_tokens:
                break
            model.tokens.copy_(nxt.view(-1).to(torch.int32))
            model.step(1)
    else:
        if max_new_tokens > 1:
            model.step(max_new_tokens - 1)
        new = model.last_tokens(max_new_tokens)[:, 0].cpu().tolist() if max_new_tokens else []
    if model.status() != 0:
        raise RuntimeError("a device-side wait ran out during generation")
    if eos is not None and int(eos) in new:
        new = new[: new.index(int(eos)) + 1]
    output_ids = input_ids[0].tolist() + new
    return {
        "prompt_token_count": prompt_len,
        "generated_token_count": len(new),
        "output_ids": output_ids,
        "completion_ids": new,
        "text": tokenizer.decode(output_ids, skip_special_tokens=False),
        "completion_text": tokenizer.decode(new, skip_special_tokens=False),
    }


def _generate_text_generic(model, tokenizer, *, prompt, max_new_tokens, device, do_sample, temperature, top_p):
    """Models without low-rank modules (anything transformers can run) take the plain token loop
    of the reference (scripts/demo_support/api.py:285-312): the model's own forward with its own
    cache, greedy or sampled.  Nothing of this library's decode path is involved."""
    dev = torch.device(device) if device is not None else next(model.parameters()).device
    enc = tokenizer(prompt, return_tensors="pt", add_special_tokens=False)
    input_ids = enc["input_ids"].to(dev)
    if int(input_ids.shape[0]) != 1:
        raise ValueError("generate_text currently supports batch_size=1 only.")
    prompt_len = int(input_ids.shape[1])
    eos = getattr(tokenizer, "eos_token_id", None)
    out = model(input_ids=input_ids, use_cache=True)
    past, logits = out.past_key_values, out.logits[:, -1, :]
    new = []
    for _ in range(int(max_new_tokens)):
        nxt = _sample_next_token(logits.float(), do_sample=do_sample, temperature=float(temperature), top_p=float(top_p))
        new.append(int(nxt[0, 0]))
        if eos is not None and new[-1] == int(eos):
            break
        out = model(input_ids=nxt, past_key_values=past, use_cache=True)
        past, logits = out.past_key_values, out.logits[:, -1, :]
    output_ids = input_ids[0].tolist() + new
    return {
        "prompt_token_count": prompt_len,
        "generated_token_count": len(new),
        "output_ids": output_ids,
        "completion_ids": new,
        "text": tokenizer.decode(output_ids, skip_special_tokens=False),
        "completion_text": tokenizer.decode(new, skip_special_tokens=False),
    }
