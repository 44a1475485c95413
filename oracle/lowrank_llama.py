"""CPU oracle: a restatement of the reference's PyTorch low-rank decode path.

TEST INFRASTRUCTURE ONLY.  Nothing in ``flashsvd_b200/`` imports this file; it is used by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` as the checker and the timed CPU baseline, never as the product path.

Parity status: PARTLY PINNED.  The reference's module file ``models/llama.py`` (the classes
``SVD_LlamaAttention`` / ``SVD_LlamaMLP`` whose fallback forward *is* the "PyTorch low-rank
path") is absent from the reference checkout (it is git-ignored there), and the reference has no
golden vectors.  What can be run from the reference is used to pin this file
(``tests/golden/make_golden.py``): its decode loop ``_manual_llama_decode_step``
(utils/evaluator.py:39-82) driving transformers' ``LlamaDecoderLayer`` / ``LlamaRMSNorm`` /
``LlamaRotaryEmbedding`` over its ``FlashSVDV15DenseKVCache`` (runtime/cache/attn_dense_kv.py),
its RoPE tables (attn_dense_kv.py:331-357), its int4 format (src/quant/packed_quant_linear.py)
and the dense-weight identity W = U·V against transformers' own dense Llama layer.

All functions take and return torch tensors and run in the dtype of their inputs, so that in
bf16 every tensor the PyTorch path materialises is rounded where that path rounds it: each
``nn.Linear`` output, the RMSNorm output, both rotary products and their sum, SiLU, the gate*up
product, the residual sums, the attention probabilities and the attention output.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

LAYER_KEYS = (
    "q_v", "q_u", "k_v", "k_u", "v_v", "v_u", "o_v", "o_u",
    "gate_v", "gate_u", "up_v", "up_u", "down_v", "down_u",
)


@dataclass
class Shape:
    """Model shape; ranks follow the reference's naming (``*_v`` input side, ``*_u`` output side)."""

    d: int = 4096
    H: int = 32
    Hk: int = 32
    Dh: int = 128
    I: int = 11008
    Rq: int = 1024
    Rk: int = 1024
    Rv: int = 1024
    Ro: int = 1024
    Rg: int = 1488
    Ru: int = 1488
    Rd: int = 1488
    vocab: int = 32000
    n_layers: int = 32
    eps: float = 1e-6
    theta: float = 10000.0

    def factor_shapes(self) -> dict[str, tuple[int, int]]:
        """nn.Linear weight shapes [out, in] of the 14 factors of a layer
        (utils/model_utils.py:637-643)."""
        d, HD, KD, I = self.d, self.H * self.Dh, self.Hk * self.Dh, self.I
        return {
            "q_v": (self.Rq, d), "q_u": (HD, self.Rq),
            "k_v": (self.Rk, d), "k_u": (KD, self.Rk),
            "v_v": (self.Rv, d), "v_u": (KD, self.Rv),
            "o_v": (self.Ro, HD), "o_u": (d, self.Ro),
            "gate_v": (self.Rg, d), "gate_u": (I, self.Rg),
            "up_v": (self.Ru, d), "up_u": (I, self.Ru),
            "down_v": (self.Rd, I), "down_u": (d, self.Rd),
        }

    def params_per_layer(self) -> int:
        return sum(a * b for a, b in self.factor_shapes().values())


LLAMA7B_SVD50 = Shape()
# Llama-2-70B shape with ~40 % of the dense parameters (80 layers, GQA 64/8)
LLAMA70B_SVD40 = Shape(d=8192, H=64, Hk=8, Dh=128, I=28672, Rq=1312, Rk=224, Rv=224, Ro=1312, Rg=2704, Ru=2704,
                       Rd=2704, vocab=32000, n_layers=80)
TINY = Shape(d=256, H=4, Hk=4, Dh=64, I=512, Rq=64, Rk=64, Rv=64, Ro=64, Rg=96, Ru=96, Rd=96,
             vocab=512, n_layers=2)
TINY_GQA = Shape(d=256, H=8, Hk=2, Dh=64, I=640, Rq=96, Rk=32, Rv=32, Ro=96, Rg=120, Ru=120,
                 Rd=120, vocab=384, n_layers=2)


# --------------------------------------------------------------------------- seeded inputs
def make_layer_weights(shape: Shape, gen: torch.Generator, dtype=torch.float32) -> dict:
    """Factors ~ N(0, 1/sqrt(fan_in)) drawn in fp32 in the fixed order of LAYER_KEYS, then cast
    (the scaling convention of the reference's own harness,
    src/legacy/FlashSVD-V1/decoders/llama/kernels/flashsvdswiglu.py:348-351); norm weights = 1."""
    w = {}
    shapes = shape.factor_shapes()
    for key in LAYER_KEYS:
        out_f, in_f = shapes[key]
        w[key] = (torch.randn(out_f, in_f, generator=gen, dtype=torch.float32) / math.sqrt(in_f)).to(dtype)
    w["ln1"] = torch.ones(shape.d, dtype=dtype)
    w["ln2"] = torch.ones(shape.d, dtype=dtype)
    return w


def make_model_weights(shape: Shape, seed: int = 0, dtype=torch.float32, n_layers: int | None = None) -> dict:
    gen = torch.Generator().manual_seed(seed)
    n = shape.n_layers if n_layers is None else n_layers
    layers = [make_layer_weights(shape, gen, dtype) for _ in range(n)]
    embed = (torch.randn(shape.vocab, shape.d, generator=gen, dtype=torch.float32) / math.sqrt(shape.d)).to(dtype)
    lm_head = (torch.randn(shape.vocab, shape.d, generator=gen, dtype=torch.float32) / math.sqrt(shape.d)).to(dtype)
    return {"layers": layers, "embed": embed, "lm_head": lm_head,
            "norm": torch.ones(shape.d, dtype=dtype)}


# --------------------------------------------------------------------------- building blocks
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """transformers LlamaRMSNorm.forward, restated by the reference at
    benchmark/mlp/bench_svd_llama_decode_graph.py:78-83: variance in fp32, cast back, then scale."""
    dt = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return weight * xf.to(dt)


def rope_tables(seqlen: int, head_dim: int, theta: float, dtype, device="cpu"):
    """cos/sin [seqlen, head_dim/2]: inv_freq = theta^(-i/half), angles in fp32, cast to the model
    dtype (runtime/cache/attn_dense_kv.py:346-356)."""
    half = head_dim // 2
    pos = torch.arange(seqlen, device=device, dtype=torch.float32)
    inv_freq = 1.0 / (float(theta) ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
    ang = torch.einsum("m,d->md", pos, inv_freq)
    return torch.cos(ang).to(dtype).contiguous(), torch.sin(ang).to(dtype).contiguous()


def rotate_half_apply(x: torch.Tensor, cos_h: torch.Tensor, sin_h: torch.Tensor) -> torch.Tensor:
    """Half-split (non-interleaved) rotary, the layout the reference passes to flash-attn
    (runtime/attn/decode_registry.py:203-204) and transformers' apply_rotary_pos_emb:
    x*cos + rotate_half(x)*sin with cos/sin = cat(half, half).  x[..., Dh], cos_h/sin_h
    broadcastable to x[..., Dh/2]."""
    cos = torch.cat([cos_h, cos_h], dim=-1)
    sin = torch.cat([sin_h, sin_h], dim=-1)
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin


def lowrank(x: torch.Tensor, v_w: torch.Tensor, u_w: torch.Tensor) -> torch.Tensor:
    """y = u_proj(v_proj(x)) (benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:116-123)."""
    return F.linear(F.linear(x, v_w), u_w)


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Single-query attention over all cached keys: softmax(q·K^T/sqrt(Dh))·V with GQA by head
    grouping (benchmark/attn/decode_compare.py:569-583, 606-622), in the operation order of
    transformers' eager attention: scores in the model dtype, softmax in fp32 cast back.
    q[H,Dh], k/v[n,Hk,Dh] -> [H,Dh]."""
    H, Dh = q.shape
    Hk = k.shape[1]
    g = H // Hk
    kk = k.permute(1, 0, 2).repeat_interleave(g, dim=0)  # [H,n,Dh]
    vv = v.permute(1, 0, 2).repeat_interleave(g, dim=0)
    scores = torch.matmul(q.unsqueeze(1), kk.transpose(1, 2)) * (1.0 / math.sqrt(Dh))  # [H,1,n]
    probs = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.matmul(probs, vv).squeeze(1)


# --------------------------------------------------------------------------- one layer, one token
def decode_layer(shape: Shape, w: dict, x: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 seqlens: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, trace: dict | None = None):
    """One decoder layer for one new token per sequence.

    x[B,d]; k_cache/v_cache[B,S_max,Hk,Dh] are updated in place at position seqlens[b]
    (keys stored after RoPE, runtime/cache/attn_dense_kv.py:7-15).  Layer structure:
    transformers LlamaDecoderLayer.forward as called from utils/evaluator.py:69-78.
    """
    B = x.shape[0]
    H, Hk, Dh = shape.H, shape.Hk, shape.Dh
    xn = rmsnorm(x, w["ln1"], shape.eps)
    p_q, p_k, p_v = F.linear(xn, w["q_v"]), F.linear(xn, w["k_v"]), F.linear(xn, w["v_v"])
    q = F.linear(p_q, w["q_u"]).view(B, H, Dh)
    k = F.linear(p_k, w["k_u"]).view(B, Hk, Dh)
    v = F.linear(p_v, w["v_u"]).view(B, Hk, Dh)
    attn = torch.empty(B, H * Dh, dtype=x.dtype)
    q_rot = torch.empty_like(q)
    for b in range(B):
        pos = int(seqlens[b])
        c, s = cos[pos].unsqueeze(0), sin[pos].unsqueeze(0)
        q_rot[b] = rotate_half_apply(q[b], c, s)
        k_cache[b, pos] = rotate_half_apply(k[b], c, s)
        v_cache[b, pos] = v[b]
        attn[b] = attend(q_rot[b], k_cache[b, : pos + 1], v_cache[b, : pos + 1]).reshape(-1)
    o = lowrank(attn, w["o_v"], w["o_u"])
    h = x + o
    hn = rmsnorm(h, w["ln2"], shape.eps)
    p_gate, p_up = F.linear(hn, w["gate_v"]), F.linear(hn, w["up_v"])
    gate, up = F.linear(p_gate, w["gate_u"]), F.linear(p_up, w["up_u"])
    act = F.silu(gate) * up  # SiLU on the rounded gate, as nn.Linear -> act_fn does
    s_rank = F.linear(act, w["down_v"])
    y = F.linear(s_rank, w["down_u"])
    out = h + y
    if trace is not None:
        trace.update(xn=xn, p_q=p_q, p_k=p_k, p_v=p_v, q=q_rot, k=k, v=v, attn=attn, o=o, h=h,
                     p_up=p_up, p_gate=p_gate, act=act, s=s_rank, y=y, out=out)
    return out


def mlp_from_pcat(pcat: torch.Tensor, w: dict) -> torch.Tensor:
    """MLP from rank space, PCat = [p_up | p_gate] (up first,
    kernels/mlp/decode/dual_split_triton_pcat_s.py:81-90)."""
    Ru = w["up_u"].shape[1]
    p_up, p_gate = pcat[:, :Ru], pcat[:, Ru:]
    act = F.silu(F.linear(p_gate, w["gate_u"])) * F.linear(p_up, w["up_u"])
    return F.linear(F.linear(act, w["down_v"]), w["down_u"])


# --------------------------------------------------------------------------- whole model
@dataclass
class DecodeState:
    k: list = field(default_factory=list)  # per layer [B,S_max,Hk,Dh]
    v: list = field(default_factory=list)
    seqlens: torch.Tensor | None = None


def new_state(shape: Shape, n_layers: int, B: int, S_max: int, dtype) -> DecodeState:
    st = DecodeState()
    for _ in range(n_layers):
        st.k.append(torch.zeros(B, S_max, shape.Hk, shape.Dh, dtype=dtype))
        st.v.append(torch.zeros(B, S_max, shape.Hk, shape.Dh, dtype=dtype))
    st.seqlens = torch.zeros(B, dtype=torch.int32)
    return st


def decode_step(shape: Shape, model: dict, tokens: torch.Tensor, st: DecodeState, cos, sin):
    """One token per sequence through embed -> layers -> norm -> lm_head
    (utils/evaluator.py:39-82).  Returns logits[B,vocab]; advances st.seqlens."""
    x = model["embed"][tokens.long()]
    for li, w in enumerate(model["layers"]):
        x = decode_layer(shape, w, x, st.k[li], st.v[li], st.seqlens, cos, sin)
    x = rmsnorm(x, model["norm"], shape.eps)
    logits = F.linear(x, model["lm_head"])
    st.seqlens += 1
    return logits


def greedy_decode(shape: Shape, model: dict, prompt: torch.Tensor, n_new: int, S_max: int | None = None):
    """Token-by-token prefill of prompt[B,L] followed by n_new greedy tokens (argmax, lowest
    index on ties, scripts/demo_support/api.py:192-194).  Returns (tokens[B,n_new], logits of
    every decode step[list of [B,vocab]], state)."""
    B, L = prompt.shape
    dtype = model["embed"].dtype
    S_max = S_max or (L + n_new + 4)
    st = new_state(shape, len(model["layers"]), B, S_max, dtype)
    cos, sin = rope_tables(S_max, shape.Dh, shape.theta, dtype)
    logits = None
    for t in range(L):
        logits = decode_step(shape, model, prompt[:, t], st, cos, sin)
    out, all_logits = [], []
    for _ in range(n_new):
        all_logits.append(logits)
        nxt = torch.argmax(logits.float(), dim=-1)
        out.append(nxt)
        logits = decode_step(shape, model, nxt, st, cos, sin)
    return torch.stack(out, dim=1), all_logits, st


# --------------------------------------------------------------------------- int4 format
def unpack_int4(packed: torch.Tensor, in_features: int) -> torch.Tensor:
    """Low nibble = even input index, high nibble = odd (src/quant/packed_quant_linear.py:18-35)."""
    lo = packed & 0x0F
    hi = (packed >> 4) & 0x0F
    out = torch.empty((packed.shape[0], packed.shape[1] * 2), dtype=torch.uint8)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out[:, :in_features]


def dequantize_int4(qweight: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, in_features: int,
                    group_size: int, dtype) -> torch.Tensor:
    """w = scale * (q - zero), groups along the input dim
    (src/quant/packed_quant_linear.py:285-300)."""
    q = unpack_int4(qweight, in_features).to(torch.float32)
    g = in_features if group_size <= 0 else group_size
    idx = torch.arange(in_features) // g
    w = scales.to(torch.float32)[:, idx] * (q - zeros.to(torch.float32)[:, idx])
    return w.to(dtype)
