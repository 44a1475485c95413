"""The drop-in boundary on the GPU: a transformers Llama whose layers hold this package's
``SVD_LlamaAttention`` / ``SVD_LlamaMLP`` is driven (a) layer by layer through
``manual_llama_decode_step`` with a ``FlashSVDV15DenseKVCache`` — the way the reference's evaluator
drives its models (utils/evaluator.py:39-82) — and (b) through ``generate_text``, which builds a
``DecodeEngine`` from the modules; both must give the CPU oracle's greedy tokens."""
import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


class _Tok:
    eos_token_id = None
    pad_token_id = 0

    def __call__(self, prompt, return_tensors="pt", add_special_tokens=False):
        return {"input_ids": torch.tensor([[int(t) for t in prompt.split()]], dtype=torch.long)}

    def decode(self, ids, skip_special_tokens=False):
        return " ".join(str(int(i)) for i in ids)


def _hf_model(shape, w, dtype, dev):
    from transformers import LlamaConfig

    from flashsvd_b200 import demo_support

    cfg = LlamaConfig(hidden_size=shape.d, num_hidden_layers=len(w["layers"]), num_attention_heads=shape.H,
                      num_key_value_heads=shape.Hk, head_dim=shape.Dh, intermediate_size=shape.I, vocab_size=shape.vocab,
                      rms_norm_eps=shape.eps, tie_word_embeddings=False, max_position_embeddings=256)
    cfg.rope_theta = shape.theta
    sd = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["norm"], "lm_head.weight": w["lm_head"]}
    for li, lw in enumerate(w["layers"]):
        for name, holder in (("q", "self_attn"), ("k", "self_attn"), ("v", "self_attn"), ("o", "self_attn"),
                             ("gate", "mlp"), ("up", "mlp"), ("down", "mlp")):
            sd[f"model.layers.{li}.{holder}.{name}_v_proj.weight"] = lw[f"{name}_v"]
            sd[f"model.layers.{li}.{holder}.{name}_u_proj.weight"] = lw[f"{name}_u"]
        sd[f"model.layers.{li}.input_layernorm.weight"] = lw["ln1"]
        sd[f"model.layers.{li}.post_attention_layernorm.weight"] = lw["ln2"]
    model = demo_support.build_svd_llama(cfg, sd)
    return demo_support.cast_model_for_inference(model, dtype="fp32" if dtype == torch.float32 else "bf16", device=dev)


@pytest.mark.parametrize("shape", [O.TINY, O.TINY_GQA])
def test_hf_layers_with_these_modules_through_the_manual_decode_step(shape):
    from flashsvd_b200 import runtime as R

    dev, dtype = torch.device("cuda:0"), torch.float32
    w = O.make_model_weights(shape, seed=4, dtype=dtype)
    model = _hf_model(shape, w, dtype, dev)
    assert type(model.model.layers[0]).__name__ == "LlamaDecoderLayer"
    prompt = torch.randint(0, shape.vocab, (2, 5), generator=torch.Generator().manual_seed(8))
    n_new = 6
    cache = R.FlashSVDV15DenseKVCache(model.config, max_batch_size=2, max_cache_len=16, device=dev, dtype=dtype)
    ids = prompt.to(dev)
    logits = None
    with torch.inference_mode():
        for t in range(prompt.shape[1]):
            out = R.manual_llama_decode_step(model, ids[:, t:t + 1], past_key_values=cache,
                                             cache_position=torch.tensor([t]))
            logits = out.logits[:, -1]
        toks = []
        for s in range(n_new):
            nxt = logits.float().argmax(-1, keepdim=True)
            toks.append(nxt[:, 0].cpu())
            out = R.manual_llama_decode_step(model, nxt, past_key_values=cache,
                                             cache_position=torch.tensor([prompt.shape[1] + s]))
            logits = out.logits[:, -1]
    ref, ref_logits, _ = O.greedy_decode(shape, w, prompt, n_new)
    assert torch.equal(torch.stack(toks, 1), ref.long())
    assert cache.get_seq_length() == prompt.shape[1] + n_new
    # a token past the end of the cache raises before anything is launched
    with torch.inference_mode(), pytest.raises(IndexError):
        R.manual_llama_decode_step(model, nxt, past_key_values=cache, cache_position=torch.tensor([16]))


def test_generate_text_builds_an_engine_from_the_modules_and_keeps_tied_factors_shared():
    from flashsvd_b200 import demo_support, engine

    dev, dtype, shape = torch.device("cuda:0"), torch.float32, O.TINY
    w = O.make_model_weights(shape, seed=1, dtype=dtype)
    # basis sharing: layer 1 uses layer 0's input-side factors
    for name in ("q_v", "k_v", "v_v", "o_v", "gate_v", "up_v", "down_v"):
        w["layers"][1][name] = w["layers"][0][name]
    model = _hf_model(shape, w, dtype, dev)
    l0, l1 = model.model.layers[0], model.model.layers[1]
    for holder, names in (("self_attn", ("q", "k", "v", "o")), ("mlp", ("gate", "up", "down"))):
        for n in names:   # tie the parameters themselves, as a basis-sharing checkpoint does
            getattr(getattr(l1, holder), f"{n}_v_proj").weight = getattr(getattr(l0, holder), f"{n}_v_proj").weight
    prompt = torch.randint(0, shape.vocab, (1, 6), generator=torch.Generator().manual_seed(2))
    text = " ".join(str(int(t)) for t in prompt[0])
    res = demo_support.generate_text(model, _Tok(), prompt=text, max_new_tokens=8)
    ref, _, _ = O.greedy_decode(shape, w, prompt, 8)
    assert res["completion_ids"] == ref[0].tolist()
    eng = engine.engine_for_model(model, batch_size=1, max_cache_len=8)
    assert eng is engine.engine_for_model(model, batch_size=1, max_cache_len=8)      # kept on the model
    for name in ("qkv_v", "upgate_v", "o_v", "down_v"):
        assert eng.layers[0][name].data_ptr() == eng.layers[1][name].data_ptr(), name
    assert eng.layers[0]["o_u"].data_ptr() != eng.layers[1]["o_u"].data_ptr()
    res2 = demo_support.generate_text(model, _Tok(), prompt=text, max_new_tokens=3)
    assert res2["completion_ids"] == ref[0].tolist()[:3]
    out = demo_support.decode_kvcache_eval(model, prompt_len=6, new_tokens=4, batch_size=1, warmup=1, max_cache_len=14)
    assert out["decode_tokens_per_s"] > 0 and out["new_tokens"] == 4


def test_kernel_level_names_of_the_reference():
    from flashsvd_b200 import runtime as R

    dev, dtype, shape = torch.device("cuda:0"), torch.bfloat16, O.TINY_GQA
    gen = torch.Generator().manual_seed(5)
    w = O.make_layer_weights(shape, gen, dtype)
    H, Hk, Dh, B = shape.H, shape.Hk, shape.Dh, 2
    lin = torch.nn.functional.linear

    def rel(a, b):
        return float((a.float().cpu() - b.float().cpu()).abs().max() / b.float().abs().max())

    # per-head bases [Hx, R, Dh], different ranks for q and k / v
    Vq = w["q_u"].reshape(H, Dh, shape.Rq).permute(0, 2, 1).contiguous().to(dev)
    Vk = w["k_u"].reshape(Hk, Dh, shape.Rk).permute(0, 2, 1).contiguous().to(dev)
    Vv = w["v_u"].reshape(Hk, Dh, shape.Rv).permute(0, 2, 1).contiguous().to(dev)
    Pq = torch.randn(B, shape.Rq, generator=gen).to(dtype)
    Pk = torch.randn(B, shape.Rk, generator=gen).to(dtype)
    Pv = torch.randn(B, shape.Rv, generator=gen).to(dtype)
    q, k, v = R.reconstruct_qkv_token_shared_hetero(Pq.to(dev), Pk.to(dev), Pv.to(dev), Vq, Vk, Vv)
    assert q.shape == (B, H, Dh) and k.shape == (B, Hk, Dh)
    assert rel(q.reshape(B, -1), lin(Pq.float(), w["q_u"].float())) <= 2e-2
    assert rel(k.reshape(B, -1), lin(Pk.float(), w["k_u"].float())) <= 2e-2
    assert rel(v.reshape(B, -1), lin(Pv.float(), w["v_u"].float())) <= 2e-2
    with pytest.raises(ValueError):
        R.reconstruct_qkv_token_shared(Pq.to(dev), Pk.to(dev), Pv.to(dev), Vq, Vk, Vv)   # ranks differ
    with pytest.raises(ValueError):
        R.reconstruct_qkv_token_shared_hetero(Pq, Pk, Pv, Vq, Vk, Vv)                     # CPU tensors
    # the reference's flash-attn call: rotary + append + attention
    S_max, ctx = 24, 10
    kc = torch.zeros(B, S_max, Hk, Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    kc[:, :ctx] = torch.randn(B, ctx, Hk, Dh, generator=gen).to(dtype)
    vc[:, :ctx] = torch.randn(B, ctx, Hk, Dh, generator=gen).to(dtype)
    cos, sin = O.rope_tables(S_max, Dh, shape.theta, dtype)
    seq = torch.full((B,), ctx, dtype=torch.int32)
    kd, vd = kc.to(dev), vc.to(dev)
    out = R.call_flash_attn_with_kvcache(None, q.view(B, 1, H, Dh), kd, vd, k_bmhd=k.view(B, 1, Hk, Dh),
                                         v_bmhd=v.view(B, 1, Hk, Dh), cache_seqlens=seq.to(dev),
                                         rotary_cos=cos.to(dev), rotary_sin=sin.to(dev), causal=True)
    assert out.shape == (B, 1, H, Dh)
    half = Dh // 2

    def rot(x, pos):
        c, s = cos[pos].float(), sin[pos].float()
        x1, x2 = x[..., :half].float(), x[..., half:].float()
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).to(dtype)

    for b in range(B):
        kq = kc[b].clone()
        vq = vc[b].clone()
        kq[ctx] = rot(k[b].cpu(), ctx)
        vq[ctx] = v[b].cpu()
        ref = O.attend(rot(q[b].cpu(), ctx), kq[:ctx + 1], vq[:ctx + 1])
        assert rel(out[b, 0], ref) <= 2e-2
        assert rel(kd[b, ctx], kq[ctx]) <= 2e-2
