"""The reference's public-API smoke checks (scripts/smoke_tests/test_public_api.py:34-85) against
this package's ``demo_support``, plus the host logic of the loaders and the cache on CPU."""
import json

import pytest
import torch

from flashsvd_b200 import demo_support
from flashsvd_b200 import runtime as R


class _TinyTokenizer:
    pad_token_id = 0
    eos_token_id = 2

    def __call__(self, text, return_tensors="pt", add_special_tokens=False):
        return {"input_ids": torch.tensor([[1, 5, 7]], dtype=torch.long),
                "attention_mask": torch.tensor([[1, 1, 1]], dtype=torch.long)}

    def decode(self, token_ids, skip_special_tokens=False):
        return " ".join(str(int(t)) for t in token_ids)


def test_public_api_exports():
    for name in ("get_model_from_local", "get_model_from_source", "decode_kvcache_eval", "configure_runtime",
                 "generate_text", "cast_model_for_inference", "load_for_inference", "runtime_env_snapshot"):
        assert callable(getattr(demo_support, name))
    for name in ("reconstruct_qkv_token", "reconstruct_qkv_token_shared", "reconstruct_qkv_token_shared_hetero",
                 "reconstruct_qkv_token_shared_prepacked", "pack_qkv_shared_bases", "call_flash_attn_with_kvcache",
                 "flashsvd_mlp_dual_split_triton_pcat_s", "FlashSVDV15DenseKVCache", "manual_llama_decode_step"):
        assert hasattr(R, name)


def test_configure_runtime_flashsvd_smoke():
    cfg = demo_support.configure_runtime(mode="flashsvd", ffn_backend="auto", enable_mlp_graph=True,
                                         mlp_graph_scope="layer_tail", enable_flash_dense_attn=True)
    assert cfg["SVDLLM_FLASH_FALLBACK"] is None
    assert cfg["FLASH_SVD_MLP_CUDA_GRAPH"] == "1"
    assert cfg["FLASH_SVD_MLP_CUDA_GRAPH_SCOPE"] == "layer_tail"
    assert cfg["FLASH_SVD_ENABLE_DENSE_ATTN_DECODE"] == "1"
    assert cfg["FLASH_SVD_DENSE_DECODE_BACKEND"] == "auto"
    assert cfg["FLASH_SVD_DENSE_DECODE_GRAPH"] == "1"
    assert cfg["FLASH_SVD_DENSE_DECODE_AUTOTUNE_SCOPE"] == "attention"


def test_generate_text_smoke_cpu():
    # a model without low-rank modules takes the plain token loop, on any device
    from transformers import GPT2Config, GPT2LMHeadModel

    model = GPT2LMHeadModel(GPT2Config(vocab_size=32, n_positions=32, n_ctx=32, n_embd=16, n_layer=2, n_head=2,
                                       bos_token_id=1, eos_token_id=2, pad_token_id=0))
    tok = _TinyTokenizer()
    tok.eos_token_id = None   # a random model may emit token 2 at once; the count below needs 4 tokens
    model = demo_support.cast_model_for_inference(model, dtype="fp32", device="cpu")
    result = demo_support.generate_text(model, tok, prompt="smoke", max_new_tokens=4, device="cpu")
    assert result["prompt_token_count"] == 3
    assert result["generated_token_count"] == 4
    assert len(result["output_ids"]) == 7
    assert len(result["completion_ids"]) == 4


def _tiny_config():
    from transformers import LlamaConfig

    return LlamaConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, head_dim=64,
                       intermediate_size=512, vocab_size=300, tie_word_embeddings=False)


def test_local_directory_round_trip(tmp_path):
    cfg = _tiny_config()
    model = demo_support.build_svd_llama(cfg)
    # ranks other than the formula's: the loader must size the modules from the state dict
    attn = model.model.layers[1].self_attn
    attn.q_v_proj, attn.q_u_proj = torch.nn.Linear(256, 40, bias=False), torch.nn.Linear(40, 256, bias=False)
    (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in cfg.to_dict().items()
                                                      if isinstance(v, (int, float, str, bool, type(None)))}))
    torch.save(model.state_dict(), tmp_path / "pytorch_model.bin")
    loaded, tok = demo_support.get_model_from_source(str(tmp_path))
    assert tok is None
    assert loaded.model.layers[1].self_attn._qkv_rank_tuple()[0] == 40
    for k, v in model.state_dict().items():
        assert torch.equal(loaded.state_dict()[k], v), k
    with pytest.raises(RuntimeError, match="not a local path"):
        demo_support.get_model_from_source("some-org/some-model")


def test_low_rank_model_on_cpu_is_refused():
    model = demo_support.build_svd_llama(_tiny_config())
    with pytest.raises(RuntimeError, match="no CPU path"):
        demo_support.generate_text(model, _TinyTokenizer(), prompt="x", max_new_tokens=2)


def test_cache_is_a_transformers_cache_with_direct_write_step():
    from transformers.cache_utils import Cache

    cfg = _tiny_config()
    cache = R.FlashSVDV15DenseKVCache(cfg, max_batch_size=2, max_cache_len=8, device="cpu", dtype=torch.float32)
    assert isinstance(cache, Cache)
    assert cache.prepare_fa2_direct_write_step(0, batch_size=2, num_heads=4, head_dim=64, q_len=2) is None
    got = cache.prepare_fa2_direct_write_step(0, batch_size=2, num_heads=4, head_dim=64, q_len=1,
                                              cache_position=torch.tensor([3]))
    kc, vc, ks, vs, sl = got
    assert kc.shape == (2, 8, 4, 64) and ks.shape == (2, 1, 4, 64)
    ks.fill_(1.0)
    assert float(cache.key_cache[0][:, 3].min()) == 1.0 and float(cache.key_cache[0][:, 2].max()) == 0.0
    assert sl.tolist() == [4, 4] and sl.dtype == torch.int32
    assert cache.prepare_fa2_direct_write_step(0, batch_size=2, num_heads=4, head_dim=64, q_len=1,
                                               cache_position=torch.tensor([1, 2])) is None
    with pytest.raises(IndexError):
        cache.prepare_fa2_direct_write_step(0, batch_size=2, num_heads=4, head_dim=64, q_len=1, cache_position=8)


def test_decode_kvcache_eval_returns_the_reference_result_keys(monkeypatch):
    """The benchmark helper's control flow and result dictionary (utils/evaluator.py:529-541) on a
    stand-in engine and stand-in CUDA events: no GPU, nothing is computed."""
    import torch

    from flashsvd_b200 import demo_support
    from flashsvd_b200.engine import DecodeEngine

    clock = {"t": 0.0}

    class Event:
        def __init__(self, enable_timing=False):
            self.t = None

        def record(self):
            self.t = clock["t"]

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    monkeypatch.setattr(torch.cuda, "Event", Event)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    eng = object.__new__(DecodeEngine)
    eng.B, eng.vocab, eng.device = 2, 50, torch.device("cpu")
    calls = []
    eng.reset = lambda: calls.append("reset")
    eng.prefill = lambda prompt: (calls.append(("prefill", tuple(prompt.shape))), clock.__setitem__("t", clock["t"] + 0.5))
    eng.step = lambda n: (calls.append(("step", n)), clock.__setitem__("t", clock["t"] + 0.01 * n))
    eng.status = lambda: 0
    with pytest.raises(NotImplementedError):
        demo_support.decode_kvcache_eval(eng, prompt_len=10, new_tokens=20, lowrank_cache=True)
    out = demo_support.decode_kvcache_eval(eng, prompt_len=10, new_tokens=20, warmup=3, flashsvd_dense_cache=True,
                                           profile_decode=False)
    assert calls == ["reset", ("prefill", (2, 10)), ("step", 3), ("step", 20)]
    assert set(out) >= {"prompt_len", "new_tokens", "batch_size", "prefill_time_s", "decode_time_s", "prefill_tok_s",
                        "decode_tok_s", "decode_ms_per_token", "lowrank_cache", "flashsvd_dense_cache", "baseline_dense_kvcache"}
    assert out["prefill_time_s"] == pytest.approx(0.5) and out["decode_time_s"] == pytest.approx(0.2)
    assert out["decode_ms_per_token"] == pytest.approx(10.0) and out["decode_tok_s"] == pytest.approx(200.0)
    assert out["prefill_tok_s"] == pytest.approx(40.0) and out["flashsvd_dense_cache"] is True
    assert out["lowrank_cache"] is False and out["baseline_dense_kvcache"] is False
