"""Whole-model parity of the programs ``bench.py`` times, at the sizes it times them.

The engine is built exactly as the benchmark builds it (``synthetic.make_engine``: 7B shape at full
width, seeded random factors, caches pre-filled with N(0,1) keys / values); its weights and caches
are copied to the host and the CPU oracle is stepped beside the GPU on the GPU's tokens
(teacher forcing), as the reference's own check does
(benchmark/decode/check_flashsvd_decode_correctness.py:213-322).

Tolerances.  fp32 mode: greedy tokens identical over 32 steps, logits rel_linf <= 1e-4 (summation
order only; the per-layer bound is 2e-5 and a layer stack adds them up).  bf16 mode: there is no
per-model bound in the reference; the per-layer bound is 2e-2, the logits after L layers are
checked against 0.1 (measured values are printed; 0.076 at 32 layers), the GPU must be no further
from an fp32-arithmetic evaluation of the same weights than the bf16 oracle is, and a token may
differ from the oracle's only where the oracle's own top-2 logit gap is within twice the logit error.
"""
import dataclasses

import pytest
import torch

from oracle import check as OC
from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from flashsvd_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")


def _engine(dev, *, dtype, n_layers, batch=1, ctx=512, share_pairs=False, factors="dense", max_new=40):
    from flashsvd_b200 import synthetic

    shape = dataclasses.replace(synthetic.LLAMA7B_SVD50, n_layers=n_layers)
    eng = synthetic.make_engine(shape, device=dev, dtype=dtype, batch=batch, ctx=ctx, max_new=max_new, seed=0,
                                share_pairs=share_pairs, factors=factors, keep_raw=(factors == "int4"))
    return eng, shape


def _report(name, res):
    rel = res["rel_linf"]
    print(f"{name}: logits rel_linf first {rel[0]:.3e} max {max(rel):.3e}; tokens equal "
          f"{res['n_equal']}/{res['n_tokens']}, all explained by the top-2 gap: {res['tokens_explained']}")


def test_config1_bf16_32_layers_teacher_forced(dev):
    """The benchmarked program itself: 32 layers, 7B shape, bf16, batch 1, 512 cached positions,
    32 greedy steps (291 stages per launch)."""
    eng, shape = _engine(dev, dtype=torch.bfloat16, n_layers=32)
    res = OC.teacher_forced(eng, shape, 32, exact_steps=3)
    assert eng.status() == 0
    eng.close()
    _report("config 1 bf16 32 layers", res)
    print("  distance from the fp32-arithmetic result on the same weights: GPU",
          [f"{v:.3e}" for v in res["rel_exact_gpu"]], "bf16 oracle", [f"{v:.3e}" for v in res["rel_exact_oracle"]])
    assert max(res["rel_linf"]) <= 0.1
    # the GPU (fp32 accumulation, bf16 at the oracle's rounding points) is no further from the
    # exact result than the bf16 oracle itself, with 50 % + 1e-2 of slack for the different order
    for g, o in zip(res["rel_exact_gpu"], res["rel_exact_oracle"]):
        assert g <= 1.5 * o + 1e-2
    assert res["tokens_explained"]
    assert res["n_equal"] >= 24   # most steps have a top-2 gap far above the bf16 error


def test_config1_fp32_8_layers_greedy_identical(dev):
    """fp32 mode at full width: identical greedy tokens over 32 steps.  8 of the 32 layers (3.2 GB of
    fp32 factors on the host for the oracle instead of 13 GB); the program has the same stage
    rotation and ring behaviour per layer as the 32-layer one."""
    eng, shape = _engine(dev, dtype=torch.float32, n_layers=8)
    res = OC.teacher_forced(eng, shape, 32)
    assert eng.status() == 0
    eng.close()
    _report("config 1 fp32 8 layers", res)
    assert res["tokens_equal"]
    assert max(res["rel_linf"]) <= 1e-4


@pytest.mark.parametrize("batch,ctx,steps", [(1, 2048, 8), (8, 2048, 4)])
def test_config2_shared_bases_bf16(dev, batch, ctx, steps):
    """Basis sharing (configuration 2): layers (2i, 2i+1) alias every input-side factor buffer;
    2048 cached positions; batch 1 and 8.  8 layers = 4 sharing pairs."""
    eng, shape = _engine(dev, dtype=torch.bfloat16, n_layers=8, batch=batch, ctx=ctx, share_pairs=True, max_new=16)
    assert eng.layers[0]["qkv_v"].data_ptr() == eng.layers[1]["qkv_v"].data_ptr()
    assert eng.layers[0]["down_v"].data_ptr() == eng.layers[1]["down_v"].data_ptr()
    assert eng.layers[0]["o_u"].data_ptr() != eng.layers[1]["o_u"].data_ptr()
    res = OC.teacher_forced(eng, shape, steps)
    assert eng.status() == 0
    eng.close()
    _report(f"config 2 shared bases B={batch} ctx={ctx}", res)
    assert max(res["rel_linf"]) <= 0.06
    assert res["tokens_explained"]


def test_config3_int4_7b_shape_model(dev):
    """int4-g128 factors with configuration 3's distributions (codes uniform in [-8, 7], fp16 scales
    uniform in [0.005, 0.02]) at the 7B shape, 4 layers, batch 1, 512 cached positions: every
    step's logits and token against the oracle on the dequantised factors."""
    eng, shape = _engine(dev, dtype=torch.bfloat16, n_layers=4, factors="int4")
    assert eng.quantized
    res = OC.teacher_forced(eng, shape, 8)
    assert eng.status() == 0
    eng.close()
    _report("config 3 int4 4 layers", res)
    assert max(res["rel_linf"]) <= 0.1
    assert res["tokens_explained"]
