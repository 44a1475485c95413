"""Host mirror of the reference's runtime surface (flashsvd_b200/runtime.py) against fixtures
produced by the reference itself (tests/golden/make_golden.py)."""
import json
import os
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from flashsvd_b200 import runtime as R

GOLD = Path(__file__).parent / "golden"


@pytest.fixture()
def clean_env():
    saved = {k: os.environ.get(k) for k in R.RUNTIME_ENV_VARS}
    yield
    for k, v in saved.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def test_configure_runtime_matches_reference_environments(clean_env):
    cases = json.loads((GOLD / "configure_runtime_cases.json").read_text())
    assert len(cases) >= 5
    for case in cases:
        assert list(case["env"].keys()) == list(R.RUNTIME_ENV_VARS)
        assert R.configure_runtime(**case["kwargs"]) == case["env"], case["kwargs"]
        assert R.runtime_env_snapshot() == case["env"]


def test_configure_runtime_rejects_unknown_mode(clean_env):
    with pytest.raises(ValueError, match="Unsupported runtime mode"):
        R.configure_runtime("turbo")


def _cache(dtype=torch.float32):
    cfg = SimpleNamespace(num_hidden_layers=2, rope_theta=10000.0)
    return R.FlashSVDV15DenseKVCache(cfg, max_batch_size=2, max_cache_len=12, device="cpu", dtype=dtype)


def test_dense_cache_scenario_matches_reference(golden):
    c = _cache()
    assert c.key_cache[0].shape == (2, 12, 0, 0)  # shaped on first use
    kk, vv = torch.from_numpy(golden["cache_k_in"]), torch.from_numpy(golden["cache_v_in"])
    for li in (0, 1):
        k, v = c.update(kk + li, vv - li, li, {"cache_position": torch.arange(5)})
        assert k.shape == (2, 2, 5, 8) and torch.equal(k, kk + li) and torch.equal(v, vv - li)
    assert np.array_equal(c.key_cache[0].numpy(), golden["cache_key0"])
    assert np.array_equal(c.value_cache[1].numpy(), golden["cache_val1"])
    assert c.get_seq_length() == int(golden["cache_seen_after_prefill"][0])
    kc, vc, sl = c.prepare_fa2_step(1, batch_size=2, cache_position=None)
    assert kc.shape == (2, 12, 2, 8) and sl.dtype == torch.int32
    assert np.array_equal(sl.numpy(), golden["cache_seqlens_none"])
    _, _, sl = c.prepare_fa2_step(1, batch_size=2, cache_position=torch.tensor([7]))
    assert np.array_equal(sl.numpy(), golden["cache_seqlens_scalar"])
    _, _, sl = c.prepare_fa2_step(0, batch_size=2, cache_position=torch.tensor([5, 3]))
    assert np.array_equal(sl.numpy(), golden["cache_seqlens_rows"])
    seen = []
    c.advance_after_fa2(1, q_len=1, cache_position=torch.tensor([5]))
    seen.append(c.get_seq_length())
    c.advance_after_fa2(0, q_len=1, cache_position=torch.tensor([5]))
    seen.append(c.get_seq_length())
    c.advance_after_fa2(0, q_len=1, cache_position=None)
    seen.append(c.get_seq_length())
    assert seen == golden["cache_seen_advances"].tolist()
    assert list(c.get_mask_sizes(torch.arange(1), 0)) == golden["cache_mask_sizes"].tolist()


def test_dense_cache_errors_and_rope_tables(golden):
    c = _cache()
    c.update(torch.zeros(1, 2, 3, 8), torch.zeros(1, 2, 3, 8), 0)
    with pytest.raises(RuntimeError, match="shape changed after init"):
        c.update(torch.zeros(1, 4, 1, 8), torch.zeros(1, 4, 1, 8), 0)
    with pytest.raises(IndexError):
        c.update(torch.zeros(1, 2, 1, 8), torch.zeros(1, 2, 1, 8), 0, {"cache_position": torch.tensor([12])})
    cos, sin = c.get_rope_tables(8, 64, device="cpu", dtype=torch.float32)
    assert np.array_equal(cos.numpy(), golden["rope_cos_f32_64"][:8]) if "rope_cos_f32_64" in golden else cos.shape == (8, 32)
    assert cos.shape == (8, 32) and sin.shape == (8, 32)
    assert c.get_rope_tables(8, 64, device="cpu", dtype=torch.float32)[0] is cos  # cached


def test_kernel_wrappers_validate_before_launch():
    # argument errors are raised before any device work, with the reference's messages
    t = torch.zeros
    with pytest.raises(AssertionError):
        R.flashsvd_mlp_dual_split_triton_pcat_s(t(1, 1, 16), t(8, 32), t(8, 32), t(32, 8), t(8, 16))
    with pytest.raises(ValueError, match="expects CUDA tensors"):
        R.pack_qkv_shared_bases(t(2, 8, 4), t(2, 8, 4), t(2, 8, 4))
    with pytest.raises(ValueError, match="expects all tensors on CUDA"):
        R.reconstruct_qkv_token_shared_prepacked(t(1, 8), t(1, 8), t(1, 8), t(8, 8), t(8, 8), t(8, 8), H=2, Hk=2, Dh=4)


def test_generate_text_needs_a_model():
    with pytest.raises(TypeError):
        R.generate_text(object(), None, prompt="x")


def test_every_name_of_the_reference_runtime_packages_is_importable():
    # runtime/attn/__init__.py:19-33, runtime/cache/__init__.py:6-10, kernels/mlp/decode/dual_split_triton.py:974-983
    names = ("call_flash_attn_with_kvcache", "get_default_flashsvd_decode_attn_mod",
             "get_default_flashsvd_attn_legacy_sparsekv_decode_mod", "get_dense_token_decode_mod",
             "get_flash_attn_with_kvcache", "get_flashsvd_decode_attn_mods", "get_flashsvd_attn_legacy_sparsekv_decode_mods",
             "get_flashsvd_v15_attn_densekv_decode_mod", "maybe_kwargs", "resolve_decode_variant",
             "resolve_legacy_sparsekv_decode_variant", "select_decode_variant", "select_legacy_sparsekv_decode_variant",
             "FlashSVDLegacySparseKVCache", "FlashSVDV15DenseKVCache", "LowRankKVCache",
             "flashsvd_mlp_dual_split_triton_v1", "flashsvd_mlp_dual_split_triton_v2", "flashsvd_mlp_dual_split_triton_v2_sm80",
             "flashsvd_mlp_dual_split_triton_v3", "flashsvd_ffn_dual_split_token", "flashsvd_ffn_dual_split_token_v2",
             "flashsvd_ffn_dual_split_token_v2_sm80", "flashsvd_ffn_dual_split_token_v3")
    for n in names:
        assert callable(getattr(R, n)), n
    mod = R.get_flashsvd_v15_attn_densekv_decode_mod()
    assert mod is R.get_dense_token_decode_mod()
    for n in ("reconstruct_qkv_token", "reconstruct_qkv_token_shared", "reconstruct_qkv_token_shared_hetero",
              "reconstruct_qkv_token_shared_prepacked", "pack_qkv_shared_bases"):
        assert callable(getattr(mod, n))
    assert R.get_flash_attn_with_kvcache() is R.flash_attn_with_kvcache
    # the rank-space path is another decode mode: its registry fails as the reference's does without its kernel files
    with pytest.raises(ImportError, match="Failed to load any decode attention module"):
        R.get_flashsvd_decode_attn_mods()
    with pytest.raises(NotImplementedError):
        R.LowRankKVCache(None, max_batch_size=1, max_cache_len=8)


def test_maybe_kwargs_and_wrapper_argument_checks():
    def f(a, b=1, *, c=2):
        return a

    assert R.maybe_kwargs(f, {"b": 3, "c": 4, "d": 5}) == {"b": 3, "c": 4}
    assert R.maybe_kwargs(len, {"x": 1}) in ({}, {"x": 1})      # builtins may hide their signature
    t = torch.zeros
    with pytest.raises(AssertionError):                          # CPU tensors are refused first, as in the reference
        R.flashsvd_mlp_dual_split_triton_v1(t(1, 1, 8), t(1, 1, 8), t(8, 32), t(8, 32), t(32, 8), t(8, 16))
    with pytest.raises(ValueError, match="only the decode call of the reference"):
        R.flash_attn_with_kvcache(t(1, 1, 2, 64), t(1, 8, 2, 64), t(1, 8, 2, 64), cache_seqlens=t(1), dropout_p=0.1)
    with pytest.raises(ValueError, match="expects CUDA tensors"):
        R.flash_attn_with_kvcache(t(1, 1, 2, 64), t(1, 8, 2, 64), t(1, 8, 2, 64), cache_seqlens=t(1))


def test_module_level_names_of_the_reference_models_module():
    # models/llama.py is absent from the reference tree; these names come from its call sites
    # (utils/model_utils.py:441-445, 768-786; benchmark/mlp/bench_real_checkpoint_mlp.py:78-86)
    from flashsvd_b200 import modules as M
    from oracle import lowrank_llama as O

    rope = M.LlamaRotaryEmbedding(64, max_position_embeddings=128, base=10000.0)
    x = torch.zeros(2, 5, 64)
    cos, sin = rope(x, torch.arange(5).expand(2, 5))
    assert cos.shape == (2, 5, 64) and torch.equal(cos[..., :32], cos[..., 32:])
    tab_c, tab_s = O.rope_tables(8, 64, 10000.0, torch.float32)         # the oracle's half-width tables
    assert torch.allclose(cos[0, :, :32], tab_c[:5], atol=1e-6) and torch.allclose(sin[1, :, :32], tab_s[:5], atol=1e-6)
    c8, _ = rope(x, seq_len=8)
    assert c8.shape == (8, 64)
    assert M.enable_flashsvd_llama_layer_tail_cuda_graph() is False
    mlp = M.SVD_LlamaMLP(64, 96, "silu", ratio=0.5)
    for name in ("_flashsvd_graph_cache", "_flashsvd_layer_graph_cache"):
        assert getattr(mlp, name) == {}
        getattr(mlp, name).clear()


def test_sampler_draws_the_reference_samplers_tokens():
    """Same seeded logits, same seeded generator: the tokens of the reference's _sample_next_token
    (scripts/demo_support/api.py:192-209), recorded by tests/golden/make_sampling_golden.py."""
    cases = json.loads((GOLD / "sampling_cases.json").read_text())
    assert len(cases) >= 7
    for c in cases:
        logits = torch.randn(3, c["vocab"], generator=torch.Generator().manual_seed(100 + c["seed"])) * 3.0
        torch.manual_seed(c["seed"])
        draws = [R._sample_next_token(logits, do_sample=c["do_sample"], temperature=c["temperature"], top_p=c["top_p"]).view(-1).tolist()
                 for _ in range(6)]
        assert draws == c["draws"], c


def test_generate_text_samples_through_the_engine_api(monkeypatch):
    """Sampled generation on a stand-in engine: logits read after every step, the drawn token written
    back as the next input, one step per token, stop at the end-of-sequence token."""
    from flashsvd_b200.engine import DecodeEngine

    eng = object.__new__(DecodeEngine)
    eng.B, eng.vocab, eng.S_max = 1, 6, 64
    state = {"logits": torch.full((1, 6), -50.0), "tokens": torch.zeros(1, dtype=torch.int32), "steps": 0, "fed": []}
    order = [4, 2, 5, 1]          # the only token with mass at each step

    def refresh():
        state["logits"].fill_(-50.0)
        state["logits"][0, order[min(state["steps"], len(order) - 1)]] = 50.0

    def step(n):
        assert n == 1
        state["fed"].append(int(state["tokens"][0]))
        state["steps"] += 1
        refresh()

    eng.reset = lambda: None
    eng.prefill = lambda ids: refresh()
    eng.step = step
    eng.status = lambda: 0
    monkeypatch.setattr(DecodeEngine, "logits", property(lambda self: state["logits"]))
    monkeypatch.setattr(DecodeEngine, "tokens", property(lambda self: state["tokens"]))

    class Tok:
        eos_token_id = 5

        def __call__(self, prompt, **kw):
            return {"input_ids": torch.tensor([[1, 2, 3]])}

        def decode(self, ids, **kw):
            return " ".join(str(i) for i in ids)

    out = R.generate_text(eng, Tok(), prompt="x", max_new_tokens=8, do_sample=True, temperature=0.7, top_p=0.9)
    assert out["completion_ids"] == [4, 2, 5]            # stops at the end-of-sequence token
    assert state["fed"] == [4, 2]                        # each drawn token became the next step's input
    assert out["output_ids"] == [1, 2, 3, 4, 2, 5] and out["generated_token_count"] == 3
