"""Low-rank Llama attention / MLP modules with the sub-module names of the reference models.

The reference's ``SVD_LlamaAttention`` / ``SVD_LlamaMLP`` (built by
src/methods/svdllm/SVDLLM_flashsvd.py:264-286, factor shapes utils/model_utils.py:637-643) hold
every projection as two bias-free ``nn.Linear`` factors: ``*_v_proj`` [d_in -> r] and ``*_u_proj``
[r -> d_out].  These classes keep that surface (names, shapes, rank formula, call signature) and
run single-token decode (one new token per sequence, CUDA tensors) through the C ABI; prompts
longer than one token take plain matmuls on the GPU, which are outside the decode path this
package accelerates.  There is no CPU compute path: CPU tensors raise.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


def svd_rank(out_features: int, in_features: int, ratio: float) -> int:
    """Rank that keeps ``ratio`` of the dense parameters: int(out * in * ratio / (out + in))
    (src/methods/svdllm/SVDLLM_flashsvd.py:286)."""
    return int(out_features * in_features * ratio / (out_features + in_features))


def _decode_ok(x: torch.Tensor) -> bool:
    if not x.is_cuda:
        raise RuntimeError("flashsvd_b200 modules run on CUDA tensors only (there is no CPU path)")
    tokens = x.shape[0] * x.shape[1]
    return x.shape[1] == 1 and x.dtype in (torch.bfloat16, torch.float32) and \
        tokens <= (8 if x.dtype == torch.bfloat16 else 4)


class _WithWorkspace(nn.Module):
    def __init__(self):
        super().__init__()
        self._ws = {}
        self._packed = {}

    def _workspace(self, x: torch.Tensor, B: int, **sizes):
        key = (str(x.device), x.dtype, B)
        ws = self._ws.get(key)
        if ws is None:
            ws = ops.make_workspace(ops.make_dims(dtype=x.dtype, B=B, **sizes), x.device)
            self._ws[key] = ws
        return ws

    def _cat(self, name: str, *linears):
        """cat of the input-side factor weights, rebuilt when one of them changes."""
        key = tuple((l.weight.data_ptr(), l.weight._version, l.weight.dtype) for l in linears)
        hit = self._packed.get(name)
        if hit is None or hit[0] != key:
            hit = (key, torch.cat([l.weight for l in linears], 0).contiguous())
            self._packed[name] = hit
        return hit[1]


class SVD_LlamaMLP(_WithWorkspace):
    def __init__(self, hidden_size: int, intermediate_size: int, hidden_act: str = "silu", ratio: float = 1.0,
                 compat_ranks: bool = False):
        super().__init__()
        if hidden_act != "silu":
            raise ValueError(f"unsupported activation {hidden_act!r} (the fused kernel computes SiLU)")
        self.hidden_size, self.intermediate_size, self.ratio = hidden_size, intermediate_size, ratio
        r = svd_rank(intermediate_size, hidden_size, ratio)
        r -= r % 8 if not compat_ranks else 0
        self.low_rank = r
        self.gate_v_proj = nn.Linear(hidden_size, r, bias=False)
        self.gate_u_proj = nn.Linear(r, intermediate_size, bias=False)
        self.up_v_proj = nn.Linear(hidden_size, r, bias=False)
        self.up_u_proj = nn.Linear(r, intermediate_size, bias=False)
        self.down_v_proj = nn.Linear(intermediate_size, r, bias=False)
        self.down_u_proj = nn.Linear(r, hidden_size, bias=False)
        # the reference keeps captured CUDA graphs of its MLP here and its benchmarks clear these
        # dicts between modes (benchmark/mlp/bench_real_checkpoint_mlp.py:78-86); nothing is captured
        # per module here (a whole model step is one launch), the dicts stay empty
        self._flashsvd_graph_cache: dict = {}
        self._flashsvd_layer_graph_cache: dict = {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, L, d = x.shape
        if _decode_ok(x):
            ws = self._workspace(x, B, d=d, I=self.intermediate_size, Ru=self.up_u_proj.in_features,
                                 Rg=self.gate_u_proj.in_features, Rd=self.down_v_proj.out_features)
            y = ops.mlp_swiglu_decode(x.reshape(B, d), self.gate_u_proj.weight, self.up_u_proj.weight,
                                      self.down_v_proj.weight, self.down_u_proj.weight, ws,
                                      upgate_v=self._cat("upgate", self.up_v_proj, self.gate_v_proj))
            return y.reshape(B, 1, d)
        gate = self.gate_u_proj(self.gate_v_proj(x))
        up = self.up_u_proj(self.up_v_proj(x))
        return self.down_u_proj(self.down_v_proj(F.silu(gate) * up))


class LlamaRotaryEmbedding(nn.Module):
    """cos / sin of the rotary embedding in the rotate-half convention, constructed as the reference's
    loaders do: ``LlamaRotaryEmbedding(head_dim, max_position_embeddings=..., base=rope_theta)``
    (utils/model_utils.py:441-445).  ``forward(x, position_ids)`` -> (cos, sin) ``[B, L, head_dim]`` in
    ``x.dtype`` with the two halves equal (the transformers layout); ``forward(x, seq_len=n)`` -> the
    first ``n`` rows ``[n, head_dim]``.  The decode kernels read the half-width tables of
    ``engine.rope_tables`` instead; this class serves code that asks the module for its embedding."""

    def __init__(self, dim: int, max_position_embeddings: int = 2048, base: float = 10000.0, device=None):
        super().__init__()
        self.dim, self.max_position_embeddings, self.base = int(dim), int(max_position_embeddings), float(base)
        inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=device) / self.dim))
        self.register_buffer("inv_freq", inv, persistent=False)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, position_ids: Optional[torch.Tensor] = None, seq_len: Optional[int] = None):
        if position_ids is None:
            n = int(seq_len) if seq_len is not None else int(x.shape[-2])
            position_ids = torch.arange(n, device=x.device)
        pos = position_ids.to(device=x.device, dtype=torch.float32)
        freqs = pos[..., None] * self.inv_freq.to(x.device)
        emb = torch.cat([freqs, freqs], dim=-1)
        return emb.cos().to(x.dtype), emb.sin().to(x.dtype)


def enable_flashsvd_llama_layer_tail_cuda_graph() -> bool:
    """The reference patches transformers' decoder layer so that the part of a layer after attention
    replays as a CUDA graph (called at import by its compression scripts and by its loaders,
    utils/model_utils.py:768-786).  Here a whole decode step is one kernel launch (or one graph
    launch for wide batches) built by ``DecodeEngine``, so there is nothing to patch: the function
    exists for callers of that name and returns False (nothing was changed)."""
    return False


def _rope_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of x[..., L, Dh] by cos/sin[L, Dh/2] (first-half angles)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


class SVD_LlamaAttention(_WithWorkspace):
    def __init__(self, config, ratio: float = 1.0, layer_idx: int = 0, compat_ranks: bool = False,
                 compat_attention: bool = False):
        super().__init__()
        self.config, self.layer_idx, self.ratio = config, int(layer_idx), ratio
        self.hidden_size = d = config.hidden_size
        self.num_heads = H = config.num_attention_heads
        self.num_key_value_heads = Hk = getattr(config, "num_key_value_heads", H)
        self.num_key_value_groups = H // Hk
        self.head_dim = Dh = getattr(config, "head_dim", None) or d // H
        self.max_position_embeddings = getattr(config, "max_position_embeddings", 2048)
        self.use_lowrank_cache = False
        # runtime caches with the reference's names (utils/model_utils.py:432-450;
        # benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:69-74 clears them by name)
        self._decode_Vq = self._decode_Vk = self._decode_Vv = self._decode_ptrs = None
        self._dense_decode_prepacked_cache: dict = {}
        self._dense_decode_backend_cache: dict = {}

        def rank(out_f, in_f):
            r = svd_rank(out_f, in_f, ratio)
            return r - (r % 8 if not compat_ranks else 0)

        self.low_rank = rq = rank(H * Dh, d)
        rk = rank(Hk * Dh, d)
        self.q_v_proj, self.q_u_proj = nn.Linear(d, rq, bias=False), nn.Linear(rq, H * Dh, bias=False)
        self.k_v_proj, self.k_u_proj = nn.Linear(d, rk, bias=False), nn.Linear(rk, Hk * Dh, bias=False)
        self.v_v_proj, self.v_u_proj = nn.Linear(d, rk, bias=False), nn.Linear(rk, Hk * Dh, bias=False)
        self.o_v_proj, self.o_u_proj = nn.Linear(H * Dh, rq, bias=False), nn.Linear(rq, d, bias=False)

    def _qkv_rank_tuple(self):
        return self.q_u_proj.in_features, self.k_u_proj.in_features, self.v_u_proj.in_features

    def _ensure_runtime_state(self) -> None:
        """(Re)creates the runtime cache attributes if a caller deleted them."""
        for name in ("_decode_Vq", "_decode_Vk", "_decode_Vv", "_decode_ptrs"):
            if not hasattr(self, name):
                setattr(self, name, None)
        for name in ("_dense_decode_prepacked_cache", "_dense_decode_backend_cache"):
            if not isinstance(getattr(self, name, None), dict):
                setattr(self, name, {})

    def _get_decode_factors(self):
        """Per-head output bases (Vq[H, Rq, Dh], Vk[Hk, Rk, Dh], Vv[Hk, Rv, Dh]): head h of
        ``q_u_proj.weight`` [H * Dh, Rq] transposed; cached until a weight changes."""
        ptrs = tuple((l.weight.data_ptr(), l.weight._version) for l in (self.q_u_proj, self.k_u_proj, self.v_u_proj))
        if self._decode_ptrs != ptrs or self._decode_Vq is None:
            H, Hk, Dh = self.num_heads, self.num_key_value_heads, self.head_dim
            self._decode_Vq = self.q_u_proj.weight.detach().view(H, Dh, -1).transpose(1, 2).contiguous()
            self._decode_Vk = self.k_u_proj.weight.detach().view(Hk, Dh, -1).transpose(1, 2).contiguous()
            self._decode_Vv = self.v_u_proj.weight.detach().view(Hk, Dh, -1).transpose(1, 2).contiguous()
            self._decode_ptrs = ptrs
        return self._decode_Vq, self._decode_Vk, self._decode_Vv

    def _get_dense_decode_tensors(self, device, dtype, past_key_value=None, cache_position=None):
        """(packed_qkv_rank[d, Rq + Rk + Rv], vq_flat[Rq, H * Dh], vk_flat[Rk, Hk * Dh],
        vv_flat[Rv, Hk * Dh], (Rq, Rk, Rv)): the operands of
        ``hidden @ packed_qkv_rank`` and ``reconstruct_qkv_token_shared_prepacked``
        (benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:101-127), cached per
        (device, dtype) until a weight changes."""
        del past_key_value, cache_position
        lin = (self.q_v_proj, self.k_v_proj, self.v_v_proj, self.q_u_proj, self.k_u_proj, self.v_u_proj)
        key = (str(device), dtype, tuple((l.weight.data_ptr(), l.weight._version) for l in lin))
        hit = self._dense_decode_prepacked_cache.get("tensors")
        if hit is None or hit[0] != key:
            def cvt(t):
                return t.detach().to(device=device, dtype=dtype)

            packed = torch.cat([cvt(self.q_v_proj.weight), cvt(self.k_v_proj.weight), cvt(self.v_v_proj.weight)], 0)
            out = (packed.t().contiguous(), cvt(self.q_u_proj.weight).t().contiguous(),
                   cvt(self.k_u_proj.weight).t().contiguous(), cvt(self.v_u_proj.weight).t().contiguous(),
                   self._qkv_rank_tuple())
            hit = (key, out)
            self._dense_decode_prepacked_cache["tensors"] = hit
        return hit[1]

    def _flashsvd_dense_decode_token_from_hidden(self, hidden_states, past_key_value, *, cache_position=None,
                                                 cache_bindings=None, advance_cache: bool = True):
        """Attention output [B, 1, d] of one new token per sequence from the (already normalised)
        hidden state [B, 1, d]: rank projection, lift, RoPE, cache append, attention over the dense
        cache and the low-rank output projection, all in the CUDA library.  ``advance_cache=False``
        leaves the cache's token count as it was (the benchmarks call the same step repeatedly,
        benchmark/attn/generate_dense_decode_plan.py:229-243)."""
        del cache_bindings
        x, cache = hidden_states, past_key_value
        B, L, d = x.shape
        if L != 1 or not _decode_ok(x):
            raise ValueError("decode path: CUDA hidden state [B, 1, d] with B <= 8 (bf16) or 4 (fp32)")
        H, Hk, Dh, li = self.num_heads, self.num_key_value_heads, self.head_dim, self.layer_idx
        cache._ensure_layer_spec(li, h=Hk, dh=Dh)
        cos, sin = cache.get_rope_tables(cache.max_cache_len, Dh, device=x.device, dtype=x.dtype)
        # a token that does not fit the cache raises, as the reference's cache does
        # (runtime/cache/attn_dense_kv.py:295-298); the position is known on the host unless the
        # caller passed a device tensor (then the kernel drops the token and flags the workspace)
        if cache_position is None:
            start = cache.get_seq_length()
        elif torch.is_tensor(cache_position):
            start = int(cache_position.max().item()) if (not cache_position.is_cuda and cache_position.numel()) else None
        else:
            start = int(cache_position)
        if start is not None and start >= cache.max_cache_len:
            raise IndexError(f"FlashSVDV15DenseKVCache write position out of range: start={start} q_len=1 "
                             f"max={cache.max_cache_len}")
        kc, vc, seqlens = cache.prepare_fa2_step(li, batch_size=B, cache_position=cache_position)
        ws = self._workspace(x, B, d=d, H=H, Hk=Hk, Dh=Dh, Rq=self.q_u_proj.in_features,
                             Rk=self.k_u_proj.in_features, Rv=self.v_u_proj.in_features,
                             Ro=self.o_v_proj.out_features, S_max=cache.max_cache_len)
        q = ops.qkv_rope_append(x.reshape(B, d), self._cat("qkv", self.q_v_proj, self.k_v_proj, self.v_v_proj),
                                self.q_u_proj.weight, self.k_u_proj.weight, self.v_u_proj.weight, cos, sin,
                                kc, vc, seqlens, ws, num_heads=H, num_kv_heads=Hk, head_dim=Dh,
                                ranks=self._qkv_rank_tuple())
        a = ops.flash_decode(q, kc, vc, seqlens, ws, seqlen_add=1)
        y = ops.lowrank_proj(a.reshape(B, H * Dh), self.o_v_proj.weight, self.o_u_proj.weight, ws)
        cache._layer_initialized[li] = True
        if advance_cache:
            cache.advance_after_fa2(li, q_len=1, cache_position=cache_position)
        return y.reshape(B, 1, d)

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids=None, past_key_values=None,
                cache_position: Optional[torch.Tensor] = None, position_embeddings=None, **kwargs):
        """Returns (attn_output[B, L, d], None) like the transformers attention protocol.
        ``past_key_values`` is a ``runtime.FlashSVDV15DenseKVCache``."""
        x, cache = hidden_states, past_key_values
        if cache is None:
            raise ValueError("SVD_LlamaAttention needs past_key_values (a FlashSVDV15DenseKVCache)")
        B, L, d = x.shape
        H, Hk, Dh, li = self.num_heads, self.num_key_value_heads, self.head_dim, self.layer_idx
        cache._ensure_layer_spec(li, h=Hk, dh=Dh)
        cos, sin = cache.get_rope_tables(cache.max_cache_len, Dh, device=x.device, dtype=x.dtype)
        if _decode_ok(x) and B == cache.max_batch_size:
            return self._flashsvd_dense_decode_token_from_hidden(x, cache, cache_position=cache_position), None
        # prompt processing: plain matmuls on the GPU, keys stored after RoPE
        if cache_position is None:
            cache_position = torch.arange(cache.get_seq_length(), cache.get_seq_length() + L, device=x.device)
        pos = cache_position.to(x.device).long()
        q = self.q_u_proj(self.q_v_proj(x)).view(B, L, H, Dh).transpose(1, 2)
        k = self.k_u_proj(self.k_v_proj(x)).view(B, L, Hk, Dh).transpose(1, 2)
        v = self.v_u_proj(self.v_v_proj(x)).view(B, L, Hk, Dh).transpose(1, 2)
        q, k = _rope_half(q, cos[pos], sin[pos]), _rope_half(k, cos[pos], sin[pos])
        kk, vv = cache.update(k, v, li, {"cache_position": pos})
        S = kk.shape[2]
        if Hk != H:
            kk = kk.repeat_interleave(H // Hk, 1)
            vv = vv.repeat_interleave(H // Hk, 1)
        mask = torch.arange(S, device=x.device)[None, :] <= pos[:, None]
        a = F.scaled_dot_product_attention(q, kk, vv, attn_mask=mask[None, None], scale=1.0 / math.sqrt(Dh))
        y = self.o_u_proj(self.o_v_proj(a.transpose(1, 2).reshape(B, L, H * Dh)))
        return y, None
