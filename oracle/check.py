"""Oracle-side checker for a whole ``DecodeEngine``: copies the engine's own weights and caches to
the host and steps the CPU oracle beside the GPU, feeding it the GPU's tokens (teacher forcing).

TEST INFRASTRUCTURE ONLY, like the rest of ``oracle/``: used by ``tests/`` and by the parity
check that ``bench.py`` runs outside its timed region; nothing in ``flashsvd_b200/`` imports it.
The comparison follows the reference's own decode check
(benchmark/decode/check_flashsvd_decode_correctness.py:213-322: teacher-forced logits and greedy
token match, rel_linf = max|ref - y| / max|ref| at :183-187).
"""
from __future__ import annotations

import torch

from . import lowrank_llama as O


def _factor_to_host(t, dtype):
    """A dense device tensor, or an int4 factor that kept its source buffers, as a host tensor in
    the model dtype (int4: dequantised as the reference does, src/quant/packed_quant_linear.py:285-300)."""
    if hasattr(t, "packed"):
        if t.raw is None:
            raise ValueError("int4 factor without its source buffers: build the engine with keep_raw=True")
        qw, sc, zr = (None if x is None else x.cpu() for x in t.raw)
        if zr is None:
            zr = torch.full_like(sc, 8, dtype=torch.int16)
        return O.dequantize_int4(qw, sc, zr, t.shape[1], 128, dtype)
    return t.detach().cpu()


def layer_weights_from_packed(pk: dict, shape: O.Shape, dtype, cache: dict | None = None) -> dict:
    """Undo ``packing.pack_layer`` / ``quant.pack_layer_q4``: the oracle's 14 factors + norm weights.
    ``cache`` maps device pointers to host copies so that tensors shared between layers (basis
    sharing) stay shared on the host."""
    cache = {} if cache is None else cache

    def host(name):
        t = pk[name]
        key = (name, t.data_ptr())
        if key not in cache:
            cache[key] = _factor_to_host(t, dtype)
        return cache[key]

    qkv_v, upgate_v = host("qkv_v"), host("upgate_v")
    Rq, Rk, Ru = shape.Rq, shape.Rk, shape.Ru
    return {
        "q_v": qkv_v[:Rq], "k_v": qkv_v[Rq:Rq + Rk], "v_v": qkv_v[Rq + Rk:],
        "q_u": host("q_u"), "k_u": host("k_u"), "v_u": host("v_u"),
        "o_v": host("o_v"), "o_u": host("o_u"),
        "up_v": upgate_v[:Ru], "gate_v": upgate_v[Ru:],
        "gate_u": host("gate_u"), "up_u": host("up_u"), "down_v": host("down_v"), "down_u": host("down_u"),
        "ln1": pk["ln1_w"].detach().cpu(), "ln2": pk["ln2_w"].detach().cpu(),
    }


def model_from_engine(eng, shape: O.Shape) -> dict:
    dtype = eng.dtype
    cache: dict = {}
    return {
        "layers": [layer_weights_from_packed(pk, shape, dtype, cache) for pk in eng.layers],
        "embed": eng.embed.detach().cpu(), "lm_head": eng.lm_head.detach().cpu(),
        "norm": eng.final_norm.detach().cpu(),
    }


def state_from_engine(eng) -> O.DecodeState:
    st = O.DecodeState()
    st.k = [k.detach().cpu().clone() for k in eng.key_cache]
    st.v = [v.detach().cpu().clone() for v in eng.value_cache]
    st.seqlens = eng.seqlens.cpu().clone()
    return st


def _layer_fp32(w: dict) -> dict:
    return {k: v.float() for k, v in w.items()}


def _decode_step_fp32(shape, model, tokens, st, cos, sin):
    """O.decode_step in fp32 arithmetic on the model's own (bf16-valued) weights, converting one
    layer at a time so that the host never holds a second copy of the whole model."""
    x = model["embed"][tokens.long()].float()
    for li, w in enumerate(model["layers"]):
        x = O.decode_layer(shape, _layer_fp32(w), x, st.k[li], st.v[li], st.seqlens, cos, sin)
    x = O.rmsnorm(x, model["norm"].float(), shape.eps)
    logits = torch.nn.functional.linear(x, model["lm_head"].float())
    st.seqlens += 1
    return logits


def teacher_forced(eng, shape: O.Shape, n_steps: int, model: dict | None = None, exact_steps: int = 0) -> dict:
    """Steps the engine n_steps times from its current state; the oracle starts from a copy of
    that state and receives the GPU's token at every step.  Returns per-step rel_linf of the
    logits, both argmax streams, and for every step the oracle's top-2 logit gap and the largest
    absolute logit difference (a token may differ only where the gap is within the error).

    exact_steps > 0 (bf16 engines): for the first steps the same layers are also evaluated in fp32
    arithmetic on the same weights ("exact").  ``rel_exact_gpu`` and ``rel_exact_oracle`` are the
    distances of the GPU and of the bf16 oracle from it: both round activations to bf16 at the
    same points, so the GPU must not be further from the exact result than the oracle is."""
    model = model_from_engine(eng, shape) if model is None else model
    st = state_from_engine(eng)
    cos, sin = O.rope_tables(eng.S_max, shape.Dh, shape.theta, eng.dtype)
    st32 = None
    if exact_steps > 0:
        st32 = O.DecodeState()
        st32.k, st32.v, st32.seqlens = [k.float() for k in st.k], [v.float() for v in st.v], st.seqlens.clone()
    rel, gap, err, tok_gpu, tok_ref, rel_eg, rel_eo = [], [], [], [], [], [], []
    for step in range(n_steps):
        tok_in = eng.tokens.cpu().clone()
        eng.step(1)
        torch.cuda.synchronize()
        lg = eng.logits.cpu().float().clone()
        tok_gpu.append(eng.tokens.cpu().long().clone())
        lr = O.decode_step(shape, model, tok_in.long(), st, cos, sin).float()
        tok_ref.append(torch.argmax(lr, dim=-1))
        rel.append(float((lg - lr).abs().max() / lr.abs().max().clamp_min(1e-30)))
        top2 = torch.topk(lr, 2, dim=-1).values
        gap.append((top2[:, 0] - top2[:, 1]))
        err.append((lg - lr).abs().max(dim=-1).values)
        if step < exact_steps:
            le = _decode_step_fp32(shape, model, tok_in, st32, cos.float(), sin.float())
            den = le.abs().max().clamp_min(1e-30)
            rel_eg.append(float((lg - le).abs().max() / den))
            rel_eo.append(float((lr - le).abs().max() / den))
    tok_gpu, tok_ref = torch.stack(tok_gpu), torch.stack(tok_ref)
    gap, err = torch.stack(gap), torch.stack(err)
    # a differing argmax is explained when the oracle's own top-2 gap is below twice the error
    explained = (tok_gpu == tok_ref) | (gap <= 2.0 * err)
    return {"rel_linf": rel, "tokens_gpu": tok_gpu, "tokens_ref": tok_ref, "gap": gap, "err": err,
            "tokens_equal": bool((tok_gpu == tok_ref).all()), "tokens_explained": bool(explained.all()),
            "n_equal": int((tok_gpu == tok_ref).sum()), "n_tokens": int(tok_gpu.numel()),
            "rel_exact_gpu": rel_eg, "rel_exact_oracle": rel_eo}
