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
