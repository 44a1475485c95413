"""Generates tests/golden/*.npz by running what can be run of the reference, and checks the oracle
against it while doing so.  Needs a FlashSVD checkout (--reference or $FLASHSVD_REFERENCE) and
transformers; run once in the build container:

    python tests/golden/make_golden.py --reference <FlashSVD checkout>

What is taken from the reference / its dependencies (nothing of it is copied into this repo):
  * utils/evaluator.py:_manual_llama_decode_step           the per-token decode loop
  * runtime/cache/attn_dense_kv.py:FlashSVDV15DenseKVCache  cache layout, update(), rope tables
  * src/quant/packed_quant_linear.py:PackedQuantLinear      int4 pack + dequantize
  * transformers LlamaForCausalLM / LlamaDecoderLayer / LlamaRMSNorm / LlamaRotaryEmbedding /
    apply_rotary_pos_emb / eager_attention_forward          the layer the reference drives
The reference's own low-rank modules (models/llama.py) are absent from its checkout, so the
attention / MLP modules plugged into the transformers layer below restate them from their call
sites: y = u_proj(v_proj(x)) per projection
(benchmark/attn/bench_real_checkpoint_decode_reconstruct.py:116-123).
"""
from __future__ import annotations

import argparse
import math
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn as nn

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import lowrank_llama as O  # noqa: E402

OUT = Path(__file__).resolve().parent


class _LowRankAttention(nn.Module):
    """q/k/v/o as two nn.Linear factors each inside the transformers attention protocol."""

    def __init__(self, config, shape: O.Shape, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.head_dim = shape.Dh
        self.num_key_value_groups = shape.H // shape.Hk
        self.scaling = shape.Dh ** -0.5
        self.attention_dropout = 0.0
        self.is_causal = True
        d, HD, KD = shape.d, shape.H * shape.Dh, shape.Hk * shape.Dh
        self.q_v_proj, self.q_u_proj = nn.Linear(d, shape.Rq, bias=False), nn.Linear(shape.Rq, HD, bias=False)
        self.k_v_proj, self.k_u_proj = nn.Linear(d, shape.Rk, bias=False), nn.Linear(shape.Rk, KD, bias=False)
        self.v_v_proj, self.v_u_proj = nn.Linear(d, shape.Rv, bias=False), nn.Linear(shape.Rv, KD, bias=False)
        self.o_v_proj, self.o_u_proj = nn.Linear(HD, shape.Ro, bias=False), nn.Linear(shape.Ro, d, bias=False)

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None,
                cache_position=None, **kwargs):
        from transformers.models.llama.modeling_llama import apply_rotary_pos_emb, eager_attention_forward

        shp = hidden_states.shape[:-1]
        hs = (*shp, -1, self.head_dim)
        q = self.q_u_proj(self.q_v_proj(hidden_states)).view(hs).transpose(1, 2)
        k = self.k_u_proj(self.k_v_proj(hidden_states)).view(hs).transpose(1, 2)
        v = self.v_u_proj(self.v_v_proj(hidden_states)).view(hs).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        if past_key_values is not None:
            k, v = past_key_values.update(k, v, self.layer_idx,
                                          {"sin": sin, "cos": cos, "cache_position": cache_position})
        out, _ = eager_attention_forward(self, q, k, v, attention_mask, dropout=0.0, scaling=self.scaling)
        out = out.reshape(*shp, -1).contiguous()
        return self.o_u_proj(self.o_v_proj(out)), None


class _LowRankMLP(nn.Module):
    def __init__(self, shape: O.Shape):
        super().__init__()
        d, I = shape.d, shape.I
        self.gate_v_proj, self.gate_u_proj = nn.Linear(d, shape.Rg, bias=False), nn.Linear(shape.Rg, I, bias=False)
        self.up_v_proj, self.up_u_proj = nn.Linear(d, shape.Ru, bias=False), nn.Linear(shape.Ru, I, bias=False)
        self.down_v_proj, self.down_u_proj = nn.Linear(I, shape.Rd, bias=False), nn.Linear(shape.Rd, d, bias=False)

    def forward(self, x):
        act = nn.functional.silu(self.gate_u_proj(self.gate_v_proj(x))) * self.up_u_proj(self.up_v_proj(x))
        return self.down_u_proj(self.down_v_proj(act))


def build_hf_model(shape: O.Shape, weights: dict, dtype):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=shape.d, intermediate_size=shape.I, num_hidden_layers=len(weights["layers"]),
                      num_attention_heads=shape.H, num_key_value_heads=shape.Hk, head_dim=shape.Dh,
                      vocab_size=shape.vocab, rms_norm_eps=shape.eps, max_position_embeddings=4096,
                      tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    cfg._attn_implementation = "eager"
    model = LlamaForCausalLM(cfg).to(dtype).eval()
    with torch.no_grad():
        model.model.embed_tokens.weight.copy_(weights["embed"])
        model.lm_head.weight.copy_(weights["lm_head"])
        model.model.norm.weight.copy_(weights["norm"])
        for li, w in enumerate(weights["layers"]):
            layer = model.model.layers[li]
            attn, mlp = _LowRankAttention(cfg, shape, li).to(dtype), _LowRankMLP(shape).to(dtype)
            for name in ("q", "k", "v", "o"):
                getattr(attn, f"{name}_v_proj").weight.copy_(w[f"{name}_v"])
                getattr(attn, f"{name}_u_proj").weight.copy_(w[f"{name}_u"])
            for name in ("gate", "up", "down"):
                getattr(mlp, f"{name}_v_proj").weight.copy_(w[f"{name}_v"])
                getattr(mlp, f"{name}_u_proj").weight.copy_(w[f"{name}_u"])
            layer.self_attn, layer.mlp = attn, mlp
            layer.input_layernorm.weight.copy_(w["ln1"])
            layer.post_attention_layernorm.weight.copy_(w["ln2"])
    return model, cfg


@torch.inference_mode()
def reference_greedy(ref_root: Path, shape: O.Shape, weights: dict, prompt: torch.Tensor, n_new: int, dtype):
    """Greedy decode through the reference's own loop and cache, one token at a time."""
    sys.path.insert(0, str(ref_root))
    from runtime.cache.attn_dense_kv import FlashSVDV15DenseKVCache
    from utils.evaluator import _manual_llama_decode_step

    class _Cache(FlashSVDV15DenseKVCache):
        # The reference pins transformers 4.57, where create_causal_mask hands get_mask_sizes the
        # cache_position tensor; the installed 5.x hands it the query length as an int.  Only
        # that argument is adapted here, the cache itself is the reference's.
        def get_mask_sizes(self, cache_position, layer_idx):
            q = int(cache_position) if isinstance(cache_position, int) else int(cache_position.shape[0])
            return q + int(self.get_seq_length()), 0

    model, cfg = build_hf_model(shape, weights, dtype)
    B, L = prompt.shape
    cache = _Cache(cfg, max_batch_size=B, max_cache_len=L + n_new + 4, device="cpu", dtype=dtype)
    logits = None
    for t in range(L):
        out = _manual_llama_decode_step(model, prompt[:, t:t + 1], past_key_values=cache,
                                        cache_position=torch.tensor([t]))
        logits = out.logits[:, -1, :]
    toks, all_logits = [], []
    for s in range(n_new):
        all_logits.append(logits.float().clone())
        nxt = logits.float().argmax(-1, keepdim=True)
        toks.append(nxt[:, 0])
        out = _manual_llama_decode_step(model, nxt, past_key_values=cache,
                                        cache_position=torch.tensor([L + s]))
        logits = out.logits[:, -1, :]
    return torch.stack(toks, 1), all_logits, cache


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FLASHSVD_REFERENCE"), required="FLASHSVD_REFERENCE" not in os.environ,
                    help="root of a FlashSVD checkout (or set FLASHSVD_REFERENCE)")
    args = ap.parse_args()
    ref = Path(args.reference)
    report = []

    # 1. rope tables: reference cache vs oracle, bit-exact
    sys.path.insert(0, str(ref))
    from runtime.cache.attn_dense_kv import FlashSVDV15DenseKVCache
    from transformers import LlamaConfig

    cfg = LlamaConfig(hidden_size=256, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=4,
                      intermediate_size=512, vocab_size=64)
    cache = FlashSVDV15DenseKVCache(cfg, max_batch_size=1, max_cache_len=8, device="cpu", dtype=torch.float32)
    rope = {}
    for dt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        for dh in (64, 128):
            c_ref, s_ref = cache.get_rope_tables(seqlen=600, head_dim=dh, device=torch.device("cpu"), dtype=dt)
            c_o, s_o = O.rope_tables(600, dh, 10000.0, dt)
            assert torch.equal(c_ref, c_o) and torch.equal(s_ref, s_o), "rope tables differ from the reference cache"
            rope[f"cos_{name}_{dh}"] = c_ref.float().numpy()[::37]
            rope[f"sin_{name}_{dh}"] = s_ref.float().numpy()[::37]
    report.append("rope tables == FlashSVDV15DenseKVCache.get_rope_tables (bit-exact, fp32+bf16, Dh 64/128)")

    # 2. greedy decode through the reference loop + cache vs the oracle
    golden = dict(rope)
    for shape_name, shape, B, L, n_new in (("tiny", O.TINY, 1, 9, 8), ("gqa", O.TINY_GQA, 2, 7, 8)):
        for dt, dname in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            w = O.make_model_weights(shape, seed=0, dtype=dt)
            prompt = torch.randint(0, shape.vocab, (B, L), generator=torch.Generator().manual_seed(123))
            r_tok, r_log, r_cache = reference_greedy(ref, shape, w, prompt, n_new, dt)
            o_tok, o_log, o_state = O.greedy_decode(shape, w, prompt, n_new, S_max=L + n_new + 4)
            tok_match = bool(torch.equal(r_tok, o_tok))
            err = max(float((a - b.float()).abs().max() / a.abs().max()) for a, b in zip(r_log, o_log))
            k_err = float((r_cache.key_cache[0][:, : L + n_new - 1].float()
                           - o_state.k[0][:, : L + n_new - 1].float()).abs().max())
            tol = 2e-5 if dt == torch.float32 else 4e-2
            assert tok_match or dt == torch.bfloat16, f"greedy tokens differ ({shape_name}, {dname})"
            assert err < tol, f"logits differ by {err} ({shape_name}, {dname})"
            report.append(f"greedy {shape_name}/{dname}: tokens equal={tok_match}, logits rel_linf={err:.2e}, "
                          f"layer-0 key cache max abs diff={k_err:.2e}")
            key = f"{shape_name}_{dname}"
            golden[f"{key}_prompt"] = prompt.numpy()
            golden[f"{key}_tokens"] = r_tok.numpy()
            golden[f"{key}_logits0"] = r_log[0].numpy()
            golden[f"{key}_logits_last"] = r_log[-1].numpy()

    # 3. dense identity: transformers' dense Llama layer with W = U V vs the oracle layer (fp32)
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding

    shape = O.TINY
    gen = torch.Generator().manual_seed(7)
    w = O.make_layer_weights(shape, gen, torch.float32)
    lcfg = LlamaConfig(hidden_size=shape.d, intermediate_size=shape.I, num_hidden_layers=1,
                       num_attention_heads=shape.H, num_key_value_heads=shape.Hk, head_dim=shape.Dh,
                       rms_norm_eps=shape.eps, attention_bias=False, mlp_bias=False)
    lcfg._attn_implementation = "eager"
    dense = LlamaDecoderLayer(lcfg, 0).eval()
    with torch.no_grad():
        for name, mod in (("q", dense.self_attn.q_proj), ("k", dense.self_attn.k_proj),
                          ("v", dense.self_attn.v_proj), ("o", dense.self_attn.o_proj),
                          ("gate", dense.mlp.gate_proj), ("up", dense.mlp.up_proj), ("down", dense.mlp.down_proj)):
            mod.weight.copy_((w[f"{name}_u"].double() @ w[f"{name}_v"].double()).float())
        dense.input_layernorm.weight.fill_(1.0)
        dense.post_attention_layernorm.weight.fill_(1.0)
    T = 6
    xs = torch.randn(1, T, shape.d, generator=gen)
    rot = LlamaRotaryEmbedding(lcfg)
    pos = torch.arange(T).unsqueeze(0)
    mask = torch.full((T, T), float("-inf")).triu(1)[None, None]
    with torch.no_grad():
        y_dense = dense(xs, attention_mask=mask, position_ids=pos, position_embeddings=rot(xs, pos))
    y_dense = y_dense[0] if isinstance(y_dense, tuple) else y_dense
    kc = torch.zeros(1, 16, shape.Hk, shape.Dh)
    vc = torch.zeros_like(kc)
    cos, sin = O.rope_tables(16, shape.Dh, shape.theta, torch.float32)
    ys = []
    for t in range(T):
        ys.append(O.decode_layer(shape, w, xs[:, t], kc, vc, torch.tensor([t], dtype=torch.int32), cos, sin))
    y_or = torch.stack(ys, 1)
    err = float((y_dense - y_or).abs().max() / y_dense.abs().max())
    assert err < 1e-4, f"oracle layer differs from the dense transformers layer by {err}"
    report.append(f"oracle layer (token by token) vs transformers dense LlamaDecoderLayer with W=U·V: rel_linf={err:.2e}")
    golden["dense_x"] = xs.numpy()
    golden["dense_y"] = y_dense.numpy()

    # 4. int4 format: reference pack + dequantize vs oracle
    sys.path.insert(0, str(ref / "src"))
    from quant.packed_quant_linear import PackedQuantLinear

    wq = torch.randn(24, 200, generator=gen)
    pq = PackedQuantLinear(in_features=200, out_features=24, bits=4, group_size=128, bias=False,
                           compute_dtype=torch.float32)
    pq.pack_weight(wq, bias=None, sym=True)
    d_ref = pq.dequantize(dtype=torch.float32)
    d_or = O.dequantize_int4(pq.qweight, pq.scales, pq.zeros, 200, 128, torch.float32)
    assert torch.equal(d_ref, d_or), "int4 dequantisation differs from PackedQuantLinear.dequantize"
    report.append("int4: oracle dequantize == PackedQuantLinear.dequantize (bit-exact, ragged last group)")
    from flashsvd_b200 import quant

    qw2, sc2, z2 = quant.quantize_symmetric(wq)
    assert torch.equal(qw2, pq.qweight) and torch.equal(sc2, pq.scales) and torch.equal(z2, pq.zeros), \
        "quant.quantize_symmetric differs from PackedQuantLinear.pack_weight(sym=True)"
    report.append("int4: quant.quantize_symmetric == PackedQuantLinear.pack_weight(sym=True) (bit-exact)")
    golden["q_weight"] = wq.numpy()
    golden["q_qweight"] = pq.qweight.numpy()
    golden["q_scales"] = pq.scales.float().numpy()
    golden["q_zeros"] = pq.zeros.numpy()
    golden["q_dequant"] = d_ref.numpy()

    # 5. host surface: configure_runtime environments and a dense-cache scenario, for the mirror
    #    in flashsvd_b200/runtime.py
    import json

    from scripts.demo_support import api

    cases = [dict(mode="flashsvd"), dict(mode="hf"), dict(mode="baseline"),
             dict(mode="FlashSVD", ffn_backend="dual-split-kernel-v2", enable_mlp_graph=False,
                  enable_flash_dense_attn=False, enable_cutlass_rope_attn=True, graph_alias_output=True,
                  mlp_graph_scope="mlp", dense_decode_backend="fa2", dense_decode_autotune_scope="layer"),
             dict(mode="flashsvd", enable_dense_decode_graph=False, dense_decode_backend="triton")]
    saved = {k: os.environ.get(k) for k in api._RUNTIME_ENV_VARS}
    env_cases = [{"kwargs": c, "env": api.configure_runtime(**c)} for c in cases]
    for k, v in saved.items():
        os.environ.pop(k, None) if v is None else os.environ.__setitem__(k, v)
    (OUT / "configure_runtime_cases.json").write_text(json.dumps(env_cases, indent=1))
    report.append(f"configure_runtime: {len(cases)} reference environments saved (15 variables each)")

    class _C2(FlashSVDV15DenseKVCache):
        def __init__(self, *a, **k):
            self._seen_tokens = 0
            super().__init__(*a, **k)
            self._seen_tokens = 0

    cfg2 = LlamaConfig(hidden_size=32, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2,
                                    intermediate_size=64, vocab_size=50, rope_theta=10000.0)
    c2 = _C2(cfg2, max_batch_size=2, max_cache_len=12, device="cpu", dtype=torch.float32)
    kk = torch.randn(2, 2, 5, 8, generator=gen)
    vv = torch.randn(2, 2, 5, 8, generator=gen)
    for li in (0, 1):
        c2.update(kk + li, vv - li, li, {"cache_position": torch.arange(5)})
    golden["cache_k_in"] = kk.numpy()
    golden["cache_v_in"] = vv.numpy()
    golden["cache_key0"] = c2.key_cache[0].numpy().copy()
    golden["cache_val1"] = c2.value_cache[1].numpy().copy()
    golden["cache_seen_after_prefill"] = np.array([c2.get_seq_length()])
    _, _, sl = c2.prepare_fa2_step(1, batch_size=2, cache_position=None)
    golden["cache_seqlens_none"] = sl.numpy().copy()
    _, _, sl = c2.prepare_fa2_step(1, batch_size=2, cache_position=torch.tensor([7]))
    golden["cache_seqlens_scalar"] = sl.numpy().copy()
    _, _, sl = c2.prepare_fa2_step(0, batch_size=2, cache_position=torch.tensor([5, 3]))
    golden["cache_seqlens_rows"] = sl.numpy().copy()
    c2.advance_after_fa2(1, q_len=1, cache_position=torch.tensor([5]))
    a1 = c2.get_seq_length()
    c2.advance_after_fa2(0, q_len=1, cache_position=torch.tensor([5]))
    a2 = c2.get_seq_length()
    c2.advance_after_fa2(0, q_len=1, cache_position=None)
    a3 = c2.get_seq_length()
    golden["cache_seen_advances"] = np.array([a1, a2, a3])
    golden["cache_mask_sizes"] = np.array(c2.get_mask_sizes(torch.arange(1), 0))
    report.append("dense cache scenario (update, prepare_fa2_step x3, advance_after_fa2 x3, get_mask_sizes) saved")

    np.savez_compressed(OUT / "reference_pins.npz", **golden)
    (OUT / "PINS.txt").write_text("\n".join(report) + "\n")
    print("\n".join(report))
    print("wrote", OUT / "reference_pins.npz")


if __name__ == "__main__":
    main()
