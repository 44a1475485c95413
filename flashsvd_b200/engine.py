"""Whole-model greedy decode on the device-resident stage program (fsvd_model_* of the C ABI).

One ``step`` is one kernel launch: embed -> all decoder layers -> final norm -> lm_head -> argmax.
Token ids and sequence lengths stay on the device between steps, which removes the per-token
``torch.tensor([pos])`` / ``.item()`` host round trips of the reference loop
(scripts/demo_support/api.py:285-312, utils/evaluator.py:499-512).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib, ops
from ._lib import FsvdLayer, LAYER_FIELDS, check


def rope_tables(seqlen: int, head_dim: int, theta: float, dtype, device):
    """cos/sin [seqlen, head_dim/2] exactly as FlashSVDV15DenseKVCache.get_rope_tables builds
    them (runtime/cache/attn_dense_kv.py:331-357): fp32 angles, cast to the model dtype."""
    half = head_dim // 2
    pos = torch.arange(seqlen, device=device, dtype=torch.float32)
    inv_freq = 1.0 / (float(theta) ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
    ang = torch.einsum("m,d->md", pos, inv_freq)
    return torch.cos(ang).to(dtype).contiguous(), torch.sin(ang).to(dtype).contiguous()


class DecodeEngine:
    """Owns the caches, the rope tables and the device program of one model replica.

    ``layers`` is a list of dicts with the tensors of ``packing.pack_layer`` (already on the
    device, model dtype).  ``k_cache`` / ``v_cache`` [B, S_max, Hk, Dh] are allocated here, one
    pair per layer, zero-initialised like the reference cache
    (runtime/cache/attn_dense_kv.py:110-130).
    """

    def __init__(self, *, layers, embed, final_norm, lm_head, num_heads, num_kv_heads, head_dim,
                 batch_size, max_cache_len, rope_theta=10000.0, eps=1e-6, max_steps=4096,
                 share_cache_alloc=True, prefill_chunk=None):
        self.lib = _lib.load()
        dev = embed.device
        if dev.type != "cuda":
            raise ValueError("flashsvd_b200 runs on CUDA devices only (there is no CPU path)")
        dtype = embed.dtype
        self.device, self.dtype = dev, dtype
        L0 = layers[0]
        d = embed.shape[1]
        H, Hk, Dh = int(num_heads), int(num_kv_heads), int(head_dim)
        Rq = L0["q_u"].shape[1]
        Rk = L0["k_u"].shape[1]
        Rv = L0["v_u"].shape[1]
        if L0["qkv_v"].shape[0] != Rq + Rk + Rv:
            raise ValueError("qkv_v rows must equal Rq + Rk + Rv")
        # int4 factors (quant.Q4Factor tile streams): bf16 everything else
        q4 = hasattr(L0["q_u"], "packed")
        if q4 and dtype != torch.bfloat16:
            raise ValueError("int4 factors need a bfloat16 model")
        self.quantized = q4
        self.dims = ops.make_dims(
            dtype=_lib.DTYPE_BF16_Q4 if q4 else dtype, B=int(batch_size), d=d, H=H, Hk=Hk, Dh=Dh, I=L0["gate_u"].shape[0],
            Rq=Rq, Rk=Rk, Rv=Rv, Ro=L0["o_v"].shape[0], Rg=L0["gate_u"].shape[1],
            Ru=L0["up_u"].shape[1], Rd=L0["down_v"].shape[0], S_max=int(max_cache_len),
            vocab=embed.shape[0], n_layers=len(layers), eps=float(eps))
        self.B, self.S_max, self.vocab, self.d = int(batch_size), int(max_cache_len), embed.shape[0], d
        self.cos, self.sin = rope_tables(self.S_max, Dh, rope_theta, dtype, dev)
        self.key_cache, self.value_cache = [], []
        # the tensors the device program points into (kept alive here)
        self.layers, self.embed, self.final_norm, self.lm_head = layers, embed, final_norm, lm_head
        arr = (FsvdLayer * len(layers))()
        for i, lw in enumerate(layers):
            kc = torch.zeros(self.B, self.S_max, Hk, Dh, dtype=dtype, device=dev)
            vc = torch.zeros_like(kc)
            self.key_cache.append(kc)
            self.value_cache.append(vc)
            t = dict(lw)
            t["k_cache"], t["v_cache"] = kc, vc
            for name in LAYER_FIELDS:
                x = t[name]
                if hasattr(x, "packed") != (q4 and name not in ("ln1_w", "ln2_w", "k_cache", "v_cache")):
                    raise ValueError(f"layer {i} tensor {name}: int4 and dense factors cannot be mixed")
                if not (x.is_cuda and x.is_contiguous() and (hasattr(x, "packed") or x.dtype == dtype)):
                    raise ValueError(f"layer {i} tensor {name}: need a contiguous {dtype} CUDA tensor")
                setattr(arr[i], name, x.data_ptr())
        for name, x in (("embed", embed), ("final_norm", final_norm), ("lm_head", lm_head)):
            if not (x.is_cuda and x.is_contiguous() and x.dtype == dtype):
                raise ValueError(f"{name}: need a contiguous {dtype} CUDA tensor")
        handle = C.c_void_p()
        with torch.cuda.device(dev):
            check(self.lib.fsvd_model_create(
                C.byref(self.dims), arr, embed.data_ptr(), final_norm.data_ptr(), lm_head.data_ptr(),
                self.cos.data_ptr(), self.sin.data_ptr(), int(max_steps), C.byref(handle)))
        self.handle = handle
        self.max_steps = int(max_steps)
        self._pos_bound = 0   # host-side upper bound of the cache positions in use
        # Prompt pass of a single sequence: a second program over the same weights and caches takes
        # `prefill_chunk` consecutive prompt positions per launch (rows_are_positions of fsvd_dims);
        # it is created on the first prompt that is long enough.
        cmax = 4 if dtype == torch.float32 else 8
        self.prefill_chunk = (cmax if prefill_chunk is None else max(1, min(int(prefill_chunk), cmax))) \
            if self.B == 1 else 1
        # long prompts of a single bf16 sequence first go 128 positions per pass through the tiled
        # tensor-core path (the same factors as 128-column GEMMs, RoPE and the cache write in their
        # epilogues, causal attention over the rows already written)
        self.prefill_tile = 128 if (self.B == 1 and dtype == torch.bfloat16 and not q4 and self.prefill_chunk > 1
                                    and self.dims.Rg == self.dims.Ru) else 0
        self._layer_array, self._model_args = arr, (embed, final_norm, lm_head)
        self._chunk_handle = None
        self._chunks: dict = {}
        ptrs = [C.c_void_p() for _ in range(6)]
        check(self.lib.fsvd_model_buffers(self.handle, *[C.byref(p) for p in ptrs]))
        self._ptrs = dict(zip(("tokens", "seqlens", "token_log", "step_counter", "logits", "hidden"),
                              (p.value for p in ptrs)))
        self.num_stages = int(self.lib.fsvd_model_num_stages(self.handle))

    # ---- device buffers as tensors (views over library-owned memory) -----------------------
    def _view(self, name, shape, dtype):
        return _from_ptr(self._ptrs[name], shape, dtype, self.device)

    @property
    def tokens(self):
        return self._view("tokens", (self.B,), torch.int32)

    @property
    def seqlens(self):
        # the caller may write through this view: the host-side position bound is no longer known
        self._pos_bound = None
        return self._view("seqlens", (self.B,), torch.int32)

    @property
    def token_log(self):
        return self._view("token_log", (self.max_steps, self.B), torch.int32)

    @property
    def step_counter(self):
        return self._view("step_counter", (1,), torch.int32)

    @property
    def logits(self):
        return self._view("logits", (self.B, self.vocab), torch.float32)

    # ---- stepping ---------------------------------------------------------------------------
    def _reserve_positions(self, n: int) -> None:
        """Raises IndexError when n more tokens do not fit the cache, as the reference's dense
        cache does (runtime/cache/attn_dense_kv.py:295-298).  The largest position is tracked on
        the host; it is read from the device (one synchronisation) only after the caller has
        touched ``seqlens``."""
        if self._pos_bound is None:
            self._pos_bound = int(self._view("seqlens", (self.B,), torch.int32).max().item())
        if self._pos_bound + n > self.S_max:
            raise IndexError(f"{n} more token(s) at position {self._pos_bound} exceed the cache "
                             f"(max_cache_len={self.S_max})")
        self._pos_bound += n

    def step(self, n_steps: int = 1) -> None:
        """Enqueue n greedy decode steps on the current stream (no synchronisation)."""
        self._reserve_positions(int(n_steps))
        check(self.lib.fsvd_model_step(self.handle, int(n_steps), torch.cuda.current_stream().cuda_stream))

    def reset(self) -> None:
        self.seqlens.zero_()
        self.step_counter.zero_()
        self._pos_bound = 0

    def _chunk_model(self, rows: Optional[int] = None):
        """The program that takes `rows` (default `prefill_chunk`) prompt positions of the one
        sequence per launch; returns (handle, tokens view, seqlens view)."""
        rows = int(self.prefill_chunk if rows is None else rows)
        hit = self._chunks.get(rows)
        if hit is None:
            d = self.dims
            dims = _lib.FsvdDims(d.dtype, rows, d.d, d.H, d.Hk, d.Dh, d.I, d.Rq, d.Rk, d.Rv, d.Ro, d.Rg, d.Ru, d.Rd,
                                 d.S_max, d.vocab, d.n_layers, d.eps, 1)
            embed, final_norm, lm_head = self._model_args
            handle = C.c_void_p()
            with torch.cuda.device(self.device):
                check(self.lib.fsvd_model_create(
                    C.byref(dims), self._layer_array, embed.data_ptr(), final_norm.data_ptr(),
                    lm_head.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), 1, C.byref(handle)))
            ptrs = [C.c_void_p() for _ in range(6)]
            check(self.lib.fsvd_model_buffers(handle, *[C.byref(p) for p in ptrs]))
            hit = (handle, _from_ptr(ptrs[0].value, (rows,), torch.int32, self.device),
                   _from_ptr(ptrs[1].value, (rows,), torch.int32, self.device), dims)
            self._chunks[rows] = hit
            if rows == self.prefill_chunk:
                self._chunk_handle, self._chunk_tokens, self._chunk_seqlens, self._chunk_dims = hit
        return hit[:3]

    def prefill(self, prompt: torch.Tensor) -> None:
        """Feed prompt[B, L] through the decode kernels: fills the caches and leaves the first
        generated token in ``tokens`` and its logits in ``logits``.  A single sequence goes 128
        positions per pass (bf16; tiled tensor-core path), then 64, 32, 16 (same path) and
        `prefill_chunk` positions per launch, causal inside a pass, each size as long as more than
        one pass of it is left, and the rest token by token; several sequences go token by token."""
        prompt = prompt.to(device=self.device, dtype=torch.int32).contiguous()
        if prompt.shape[0] != self.B:
            raise ValueError(f"prompt batch {prompt.shape[0]} != engine batch {self.B}")
        L, t0 = prompt.shape[1], 0
        tiles = (128, 64, 32, 16) if self.prefill_tile else ()
        sizes = [c for c in (*tiles, self.prefill_chunk) if c > 1 and L > c]
        if self.B == 1 and sizes:
            pos0 = int(self.seqlens[0].item())
            if pos0 + L > self.S_max:
                raise ValueError(f"prompt of {L} tokens at position {pos0} exceeds the cache ({self.S_max})")
            stream = torch.cuda.current_stream().cuda_stream
            for Cn in sizes:
                if L - t0 <= Cn:
                    continue
                handle, tokens, seqlens = self._chunk_model(Cn)
                offs = torch.arange(Cn, device=self.device, dtype=torch.int32)
                while L - t0 > Cn:
                    tokens.copy_(prompt[0, t0:t0 + Cn])
                    seqlens.copy_(offs + (pos0 + t0))
                    check(self.lib.fsvd_model_step(handle, 1, stream))
                    t0 += Cn
            self.seqlens.fill_(pos0 + t0)
            self._pos_bound = pos0 + t0
        tok = self.tokens
        for t in range(t0, L):
            tok.copy_(prompt[:, t])
            self.step(1)

    def last_tokens(self, n: int) -> torch.Tensor:
        """The tokens sampled by the last n single-token launches, [n, B] (blocking).  After
        ``prefill`` + ``step(n - 1)`` these are the n generated tokens."""
        steps = int(self.step_counter.item())
        if n > steps or steps > self.max_steps:
            raise IndexError(f"{n} tokens asked, {steps} logged (log capacity {self.max_steps})")
        return self.token_log[steps - n: steps].clone()

    def status(self) -> int:
        st = C.c_int(0)
        check(self.lib.fsvd_model_status(self.handle, C.byref(st)))
        for hit in self._chunks.values():
            if st.value == 0:
                check(self.lib.fsvd_model_status(hit[0], C.byref(st)))
        return int(st.value)

    def close(self) -> None:
        for hit in getattr(self, "_chunks", {}).values():
            if hit[0].value:
                self.lib.fsvd_model_destroy(hit[0])
        self._chunks = {}
        self._chunk_handle = None
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.fsvd_model_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _from_ptr(ptr: int, shape, dtype, device) -> torch.Tensor:
    """Wrap library-owned device memory as a tensor without copying (CUDA array interface)."""
    typestr = {torch.int32: "<i4", torch.float32: "<f4", torch.int64: "<i8", torch.uint8: "|u1"}[dtype]

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {
        "shape": tuple(int(s) for s in shape), "typestr": typestr, "data": (int(ptr), False),
        "version": 2, "strides": None,
    }
    with torch.cuda.device(device):
        return torch.as_tensor(h, device=device)


# ---- engines for transformers models that hold low-rank modules ---------------------------------
_FACTOR_NAMES = (("q", "self_attn"), ("k", "self_attn"), ("v", "self_attn"), ("o", "self_attn"),
                 ("gate", "mlp"), ("up", "mlp"), ("down", "mlp"))


def has_lowrank_modules(model) -> bool:
    """True for a Llama-shaped transformers model whose layers hold ``*_v_proj`` / ``*_u_proj``
    factor pairs (the reference's SVD_LlamaAttention / SVD_LlamaMLP, utils/model_utils.py:637-643)."""
    layers = getattr(getattr(model, "model", None), "layers", None)
    if not layers:
        return False
    attn, mlp = getattr(layers[0], "self_attn", None), getattr(layers[0], "mlp", None)
    return hasattr(attn, "q_u_proj") and hasattr(attn, "q_v_proj") and hasattr(mlp, "gate_u_proj")


def engine_for_model(model, *, batch_size: int = 1, max_cache_len: int = 2048, max_steps: int = 4096):
    """A ``DecodeEngine`` over the weights of ``model`` (a transformers LlamaForCausalLM whose
    layers hold low-rank modules), built once and kept on the model; a longer cache or another
    batch size builds a new one.  Factor weights are packed into the kernels' layout; ``*_v_proj``
    weights that several layers share (basis sharing: the same storage) are packed once and shared
    by those layers in the engine too."""
    from . import packing

    if not has_lowrank_modules(model):
        raise TypeError("the model has no *_v_proj / *_u_proj factor modules")
    emb = model.model.embed_tokens.weight
    if not emb.is_cuda:
        raise RuntimeError("flashsvd_b200 runs on CUDA tensors only (there is no CPU path): move the model to a GPU")
    key = (int(batch_size), str(emb.device), emb.dtype)
    cached = getattr(model, "_flashsvd_b200_engines", None)
    if cached is None:
        cached = {}
        object.__setattr__(model, "_flashsvd_b200_engines", cached)
    eng = cached.get(key)
    if eng is not None and eng.S_max >= int(max_cache_len):
        return eng
    if eng is not None:
        eng.close()
    cfg = model.config
    dev, dtype = emb.device, emb.dtype
    shared: dict = {}

    def once(t):   # one device copy per storage: tied input-side factors stay one buffer
        k = (t.data_ptr(), tuple(t.shape))
        if k not in shared:
            shared[k] = t.detach()
        return shared[k]

    packed_v: dict = {}
    layers = []
    for layer in model.model.layers[: cfg.num_hidden_layers]:
        w = {"ln1": layer.input_layernorm.weight, "ln2": layer.post_attention_layernorm.weight}
        for name, holder in _FACTOR_NAMES:
            mod = getattr(layer, holder)
            w[f"{name}_v"] = once(getattr(mod, f"{name}_v_proj").weight)
            w[f"{name}_u"] = once(getattr(mod, f"{name}_u_proj").weight)
        pk = packing.pack_layer(w, device=dev, dtype=dtype)
        # the concatenated input-side factors of layers that tie all of their parts are shared too
        for cat_name, parts in (("qkv_v", ("q_v", "k_v", "v_v")), ("upgate_v", ("up_v", "gate_v"))):
            k = tuple(w[p_].data_ptr() for p_ in parts)
            if k in packed_v:
                pk[cat_name] = packed_v[k]
            else:
                packed_v[k] = pk[cat_name]
        for single in ("o_v", "down_v"):
            k = (w[single].data_ptr(),)
            if k in packed_v:
                pk[single] = packed_v[k]
            else:
                packed_v[k] = pk[single]
        layers.append(pk)
    H = cfg.num_attention_heads
    eng = DecodeEngine(layers=layers, embed=emb.detach().contiguous(),
                       final_norm=model.model.norm.weight.detach().contiguous(),
                       lm_head=model.lm_head.weight.detach().contiguous(), num_heads=H,
                       num_kv_heads=getattr(cfg, "num_key_value_heads", H),
                       head_dim=getattr(cfg, "head_dim", None) or cfg.hidden_size // H, batch_size=int(batch_size),
                       max_cache_len=int(max_cache_len), rope_theta=_rope_theta(cfg),
                       eps=float(getattr(cfg, "rms_norm_eps", 1e-6)), max_steps=int(max_steps))
    cached[key] = eng
    return eng


def _rope_theta(cfg) -> float:
    theta = getattr(cfg, "rope_theta", None)
    if theta is None:
        rp = getattr(cfg, "rope_parameters", None) or {}
        theta = rp.get("rope_theta", 10000.0) if isinstance(rp, dict) else 10000.0
    return float(theta)


class EngineGroup:
    """Several ``DecodeEngine``s over the same factor tensors, each with its own caches and at most
    ``width`` sequences: how a batch runs that is wider than the kernel family of its factor type
    takes in one launch (int4 and fp32 factors have no tiled path: 8 and 4 sequences per launch).
    A step launches every engine once on the current stream; the factors are streamed once per
    engine.  The interface is the subset of ``DecodeEngine`` that decoding needs."""

    def __init__(self, *, batch_size: int, width: int, **engine_kwargs):
        if batch_size < 1 or width < 1:
            raise ValueError("batch_size and width must be positive")
        sizes = [width] * (batch_size // width) + ([batch_size % width] if batch_size % width else [])
        self.engines = [DecodeEngine(batch_size=b, **engine_kwargs) for b in sizes]
        self.B = int(batch_size)
        e0 = self.engines[0]
        self.S_max, self.vocab, self.device, self.quantized = e0.S_max, e0.vocab, e0.device, e0.quantized
        self.key_cache = [[e.key_cache[l] for e in self.engines] for l in range(len(e0.key_cache))]
        self.value_cache = [[e.value_cache[l] for e in self.engines] for l in range(len(e0.value_cache))]

    @property
    def tokens(self) -> torch.Tensor:
        """A copy of the current tokens of all sequences (write through ``set_tokens``)."""
        return torch.cat([e.tokens for e in self.engines])

    def set_tokens(self, tokens: torch.Tensor) -> None:
        o = 0
        for e in self.engines:
            e.tokens.copy_(tokens[o:o + e.B])
            o += e.B

    def fill_seqlens(self, value: int) -> None:
        for e in self.engines:
            e.seqlens.fill_(int(value))
            e._pos_bound = int(value)

    def step(self, n_steps: int = 1) -> None:
        for _ in range(int(n_steps)):
            for e in self.engines:
                e.step(1)

    def prefill(self, prompt: torch.Tensor) -> None:
        o = 0
        for e in self.engines:
            e.prefill(prompt[o:o + e.B])
            o += e.B

    def last_tokens(self, n: int) -> torch.Tensor:
        return torch.cat([e.last_tokens(n) for e in self.engines], dim=1)

    def status(self) -> int:
        for e in self.engines:
            st = e.status()
            if st:
                return st
        return 0

    def close(self) -> None:
        for e in self.engines:
            e.close()
