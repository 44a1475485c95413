"""CPU: the oracle against the golden vectors produced by running the reference's decode loop,
cache, rope tables and int4 format (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import lowrank_llama as O

CASES = [("tiny", O.TINY, 9, 8), ("gqa", O.TINY_GQA, 7, 8)]


@pytest.mark.parametrize("name,shape,L,n_new", CASES)
def test_fp32_greedy_is_bit_identical_to_reference_loop(golden, name, shape, L, n_new):
    w = O.make_model_weights(shape, seed=0, dtype=torch.float32)
    prompt = torch.from_numpy(golden[f"{name}_f32_prompt"])
    toks, logits, _ = O.greedy_decode(shape, w, prompt, n_new, S_max=L + n_new + 4)
    assert np.array_equal(toks.numpy(), golden[f"{name}_f32_tokens"])
    assert np.array_equal(logits[0].numpy(), golden[f"{name}_f32_logits0"])
    assert np.array_equal(logits[-1].numpy(), golden[f"{name}_f32_logits_last"])


@pytest.mark.parametrize("name,shape,L,n_new", CASES)
def test_bf16_greedy_matches_reference_loop(golden, name, shape, L, n_new):
    w = O.make_model_weights(shape, seed=0, dtype=torch.bfloat16)
    prompt = torch.from_numpy(golden[f"{name}_bf16_prompt"])
    toks, logits, _ = O.greedy_decode(shape, w, prompt, n_new, S_max=L + n_new + 4)
    assert np.array_equal(toks.numpy(), golden[f"{name}_bf16_tokens"])
    ref = golden[f"{name}_bf16_logits0"]
    rel = np.abs(logits[0].float().numpy() - ref).max() / np.abs(ref).max()
    assert rel <= 2e-2  # bf16 tolerance of the decode path: per-layer max relative error


def test_rope_tables_match_reference_cache(golden):
    for dt, name in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        for dh in (64, 128):
            c, s = O.rope_tables(600, dh, 10000.0, dt)
            assert np.array_equal(c.float().numpy()[::37], golden[f"cos_{name}_{dh}"])
            assert np.array_equal(s.float().numpy()[::37], golden[f"sin_{name}_{dh}"])


def test_int4_dequantize_matches_reference(golden):
    q = torch.from_numpy(golden["q_qweight"])
    sc = torch.from_numpy(golden["q_scales"]).to(torch.float16)
    z = torch.from_numpy(golden["q_zeros"])
    d = O.dequantize_int4(q, sc, z, 200, 128, torch.float32)
    assert np.array_equal(d.numpy(), golden["q_dequant"])


def test_int4_quantiser_matches_reference(golden):
    # flashsvd_b200.quant.quantize_symmetric against PackedQuantLinear.pack_weight(sym=True)
    # (src/quant/packed_quant_linear.py:126-171): codes, fp16 scales and zero points bit-exact
    from flashsvd_b200 import quant

    qw, sc, z = quant.quantize_symmetric(torch.from_numpy(golden["q_weight"]))
    assert np.array_equal(qw.numpy(), golden["q_qweight"])
    assert np.array_equal(sc.float().numpy(), golden["q_scales"])
    assert np.array_equal(z.numpy(), golden["q_zeros"])


def test_layer_matches_dense_transformers_layer(golden):
    shape = O.TINY
    gen = torch.Generator().manual_seed(7)
    w = O.make_layer_weights(shape, gen, torch.float32)
    xs = torch.from_numpy(golden["dense_x"])
    kc = torch.zeros(1, 16, shape.Hk, shape.Dh)
    vc = torch.zeros_like(kc)
    cos, sin = O.rope_tables(16, shape.Dh, shape.theta, torch.float32)
    ys = [O.decode_layer(shape, w, xs[:, t], kc, vc, torch.tensor([t], dtype=torch.int32), cos, sin)
          for t in range(xs.shape[1])]
    y = torch.stack(ys, 1).numpy()
    ref = golden["dense_y"]
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-4


def test_empty_cache_first_token_and_param_count():
    shape = O.TINY
    w = O.make_model_weights(shape, seed=1, dtype=torch.float32)
    toks, logits, st = O.greedy_decode(shape, w, torch.tensor([[5]]), 1)
    assert int(st.seqlens[0]) == 2 and toks.shape == (1, 1)
    assert O.LLAMA7B_SVD50.params_per_layer() == 100_978_688
