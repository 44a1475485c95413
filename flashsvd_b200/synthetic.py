"""Seeded synthetic models with the shapes of the benchmark configurations.

The reference measures on real checkpoints that are not available offline; the benchmark and the
large-shape tests use random factors of the same shapes instead: N(0, 1/sqrt(fan_in)) factors,
unit RMSNorm weights, the scaling of the reference's own kernel harness
(src/legacy/FlashSVD-V1/decoders/llama/kernels/flashsvdswiglu.py:348-351).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class ModelShape:
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

    def params_per_layer(self) -> int:
        d, HD, KD, I = self.d, self.H * self.Dh, self.Hk * self.Dh, self.I
        return (d * self.Rq + HD * self.Rq + d * self.Rk + KD * self.Rk + d * self.Rv + KD * self.Rv
                + HD * self.Ro + d * self.Ro + d * self.Rg + I * self.Rg + d * self.Ru + I * self.Ru
                + I * self.Rd + d * self.Rd)

    def bytes_per_step(self, ctx: int, batch: int, esize: int = 2) -> int:
        """Algorithmic HBM bytes of one decode step: every factor once, the K and V rows of the
        context, lm_head once."""
        kv = 2 * batch * ctx * self.Hk * self.Dh * esize
        return self.n_layers * (self.params_per_layer() * esize + kv) + self.vocab * self.d * esize

    def factor_dims(self):
        """(rows, in_features) of the 14 factors of a layer."""
        d, HD, KD, I = self.d, self.H * self.Dh, self.Hk * self.Dh, self.I
        return [(self.Rq, d), (HD, self.Rq), (self.Rk, d), (KD, self.Rk), (self.Rv, d), (KD, self.Rv),
                (self.Ro, HD), (d, self.Ro), (self.Rg, d), (I, self.Rg), (self.Ru, d), (I, self.Ru),
                (self.Rd, I), (d, self.Rd)]

    def q4_bytes_per_layer(self, group: int = 128) -> int:
        """Algorithmic bytes of a layer's int4-g128 factors: half a byte per code and one fp16
        scale per row and group."""
        return sum(r * k // 2 + r * ((k + group - 1) // group) * 2 for r, k in self.factor_dims())

    def q4_bytes_per_step(self, ctx: int, batch: int) -> int:
        kv = 2 * batch * ctx * self.Hk * self.Dh * 2
        return self.n_layers * (self.q4_bytes_per_layer() + kv) + self.vocab * self.d * 2


LLAMA7B_SVD50 = ModelShape()
# Llama-2-70B shape with ~40 % of the dense parameters: 55 GB of bf16 factors, one replica fits a GPU
LLAMA70B_SVD40 = ModelShape(d=8192, H=64, Hk=8, Dh=128, I=28672, Rq=1312, Rk=224, Rv=224, Ro=1312, Rg=2704,
                            Ru=2704, Rd=2704, vocab=32000, n_layers=80)


def _qkv_u(w, HD, KD, shape):
    """q_u / k_u / v_u, back to back in one allocation when the ranks agree (packing.pack_layer)."""
    if shape.Rq == shape.Rk == shape.Rv:
        t = w(HD + 2 * KD, shape.Rq)
        t[HD:] *= 1.0   # same distribution for all three parts
        return {"q_u": t[:HD], "k_u": t[HD:HD + KD], "v_u": t[HD + KD:]}
    return {"q_u": w(HD, shape.Rq), "k_u": w(KD, shape.Rk), "v_u": w(KD, shape.Rv)}


def random_packed_layers(shape: ModelShape, *, device, dtype, seed: int = 0, share_pairs: bool = False):
    """Per-layer tensors in the layout of ``packing.pack_layer``, drawn directly on the device.
    ``share_pairs``: layers (2i, 2i+1) share every input-side factor tensor (basis sharing,
    utils/model_utils.py:366-406)."""
    gen = torch.Generator(device=device).manual_seed(seed)

    def w(out_f, in_f):
        t = torch.randn(out_f, in_f, device=device, dtype=torch.float32, generator=gen)
        return (t / math.sqrt(in_f)).to(dtype)

    d, HD, KD, I = shape.d, shape.H * shape.Dh, shape.Hk * shape.Dh, shape.I
    layers = []
    for li in range(shape.n_layers):
        if share_pairs and li % 2 == 1:
            prev = layers[-1]
            qkv_v, o_v, upgate_v, down_v = prev["qkv_v"], prev["o_v"], prev["upgate_v"], prev["down_v"]
        else:
            qkv_v = w(shape.Rq + shape.Rk + shape.Rv, d)
            o_v = w(shape.Ro, HD)
            upgate_v = w(shape.Ru + shape.Rg, d)
            down_v = w(shape.Rd, I)
        layers.append({
            "ln1_w": torch.ones(d, device=device, dtype=dtype),
            "qkv_v": qkv_v, **_qkv_u(w, HD, KD, shape),
            "o_v": o_v, "o_u": w(d, shape.Ro),
            "ln2_w": torch.ones(d, device=device, dtype=dtype),
            "upgate_v": upgate_v, "gate_u": w(I, shape.Rg), "up_u": w(I, shape.Ru),
            "down_v": down_v, "down_u": w(d, shape.Rd),
        })
    embed = w(shape.vocab, d)
    lm_head = w(shape.vocab, d)
    final_norm = torch.ones(d, device=device, dtype=dtype)
    return layers, embed, final_norm, lm_head


def random_q4_layers(shape: ModelShape, *, device, seed: int = 0, scale_lo: float = 0.005, scale_hi: float = 0.02,
                     keep_raw: bool = False):
    """Per-layer int4-g128 factors as tile streams (quant.pack_layer_q4), drawn on the device:
    codes uniform in [-8, 7], fp16 scales uniform in [scale_lo, scale_hi]; dense bf16 embedding,
    lm_head and unit norm weights."""
    from . import quant
    from .packing import FACTOR_KEYS

    gen = torch.Generator(device=device).manual_seed(seed)
    d, HD, KD, I = shape.d, shape.H * shape.Dh, shape.Hk * shape.Dh, shape.I
    dims = {"q_v": (shape.Rq, d), "q_u": (HD, shape.Rq), "k_v": (shape.Rk, d), "k_u": (KD, shape.Rk),
            "v_v": (shape.Rv, d), "v_u": (KD, shape.Rv), "o_v": (shape.Ro, HD), "o_u": (d, shape.Ro),
            "gate_v": (shape.Rg, d), "gate_u": (I, shape.Rg), "up_v": (shape.Ru, d), "up_u": (I, shape.Ru),
            "down_v": (shape.Rd, I), "down_u": (d, shape.Rd)}
    layers = []
    for _ in range(shape.n_layers):
        q = {}
        for key in FACTOR_KEYS:
            out_f, in_f = dims[key]
            q[key] = (*quant.random_q4(out_f, in_f, generator=gen, device=device, scale_lo=scale_lo,
                                       scale_hi=scale_hi), in_f)
        ones = torch.ones(d, device=device, dtype=torch.bfloat16)
        layers.append(quant.pack_layer_q4(q, ln1=ones, ln2=ones.clone(), keep_raw=keep_raw))

    def w(out_f, in_f):
        t = torch.randn(out_f, in_f, device=device, dtype=torch.float32, generator=gen)
        return (t / math.sqrt(in_f)).to(torch.bfloat16)

    return layers, w(shape.vocab, d), torch.ones(d, device=device, dtype=torch.bfloat16), w(shape.vocab, d)


def make_engine(shape: ModelShape, *, device, dtype=torch.bfloat16, batch=1, ctx=512, max_new=64, seed=0,
                fill_cache=True, share_pairs=False, factors="dense", keep_raw=False):
    """Random model + engine whose caches already hold ``ctx`` tokens of N(0,1) keys / values (the
    state after a prefill of that length, as far as the cost of a decode step goes)."""
    from .engine import DecodeEngine

    if factors == "int4":
        layers, embed, final_norm, lm_head = random_q4_layers(shape, device=device, seed=seed, keep_raw=keep_raw)
    else:
        layers, embed, final_norm, lm_head = random_packed_layers(shape, device=device, dtype=dtype, seed=seed,
                                                                  share_pairs=share_pairs)
    width = 8 if factors == "int4" else (4 if dtype == torch.float32 else 128)
    if batch > width:
        # wider than one launch of this factor type takes: a group of engines over the same factors
        from .engine import EngineGroup

        grp = EngineGroup(batch_size=batch, width=width, layers=layers, embed=embed, final_norm=final_norm,
                          lm_head=lm_head, num_heads=shape.H, num_kv_heads=shape.Hk, head_dim=shape.Dh,
                          max_cache_len=ctx + max_new + 4, rope_theta=shape.theta, eps=shape.eps, max_steps=max_new + 8)
        if fill_cache and ctx > 0:
            gen = torch.Generator(device=device).manual_seed(seed + 1)
            for e in grp.engines:
                for kc, vc in zip(e.key_cache, e.value_cache):
                    kc[:, :ctx].copy_(torch.randn(kc[:, :ctx].shape, device=device, generator=gen).to(dtype))
                    vc[:, :ctx].copy_(torch.randn(vc[:, :ctx].shape, device=device, generator=gen).to(dtype))
            grp.fill_seqlens(ctx)
        grp.set_tokens(torch.arange(batch, device=device, dtype=torch.int32) % shape.vocab)
        return grp
    eng = DecodeEngine(layers=layers, embed=embed, final_norm=final_norm, lm_head=lm_head,
                       num_heads=shape.H, num_kv_heads=shape.Hk, head_dim=shape.Dh, batch_size=batch,
                       max_cache_len=ctx + max_new + 4, rope_theta=shape.theta, eps=shape.eps,
                       max_steps=max_new + 8)
    if fill_cache and ctx > 0:
        gen = torch.Generator(device=device).manual_seed(seed + 1)
        for kc, vc in zip(eng.key_cache, eng.value_cache):
            kc[:, :ctx].copy_(torch.randn(kc[:, :ctx].shape, device=device, generator=gen).to(dtype))
            vc[:, :ctx].copy_(torch.randn(vc[:, :ctx].shape, device=device, generator=gen).to(dtype))
        eng.seqlens.fill_(ctx)
        eng._pos_bound = int(ctx)   # known on the host: no device read at the first step
    eng.tokens.copy_(torch.arange(batch, device=device, dtype=torch.int32) % shape.vocab)
    if not (fill_cache and ctx > 0):
        eng._pos_bound = 0
    return eng
