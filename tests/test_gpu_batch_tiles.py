"""Batches of 9..128 sequences: the tiled tensor-core path (tcgen05 GEMMs with the accumulators in
tensor memory, `flashsvd_b200/csrc/fsvd_tile.cu`) against the CPU oracle, through the same C entry
points as the small batches (`fsvd_decode_layer`, `fsvd_model_*` with `fsvd_dims.B` > 8).

Tolerance: the bf16 per-layer bound 2e-2 (rel_linf), as for the small batches."""
import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from flashsvd_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")


def rel_linf(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def _layer_case(dev, shape, B, ctx, S_max, seed=0, ragged=True):
    from flashsvd_b200 import ops, packing

    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(seed)
    w = O.make_layer_weights(shape, gen, dtype)
    x = torch.randn(B, shape.d, generator=gen).to(dtype)
    kc = torch.zeros(B, S_max, shape.Hk, shape.Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    kc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen).to(dtype)
    vc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen).to(dtype)
    seqlens = torch.full((B,), ctx, dtype=torch.int32)
    if ragged:
        for b in range(B):
            seqlens[b] = max(0, ctx - 3 * (b % 5))   # ragged batch, one sequence possibly short
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    kc_o, vc_o = kc.clone(), vc.clone()
    ref = O.decode_layer(shape, w, x, kc_o, vc_o, seqlens, cos, sin)
    pk = packing.pack_layer(w, device=dev, dtype=dtype)
    pk["k_cache"], pk["v_cache"] = kc.to(dev), vc.to(dev)
    dims = ops.make_dims(dtype=dtype, B=B, d=shape.d, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, I=shape.I, Rq=shape.Rq,
                         Rk=shape.Rk, Rv=shape.Rv, Ro=shape.Ro, Rg=shape.Rg, Ru=shape.Ru, Rd=shape.Rd,
                         S_max=S_max, eps=shape.eps)
    ws = ops.make_workspace(dims, dev)
    out = torch.empty(B, shape.d, dtype=dtype, device=dev)
    xd = x.to(dev)
    ops.decode_layer(dims, ops.make_layer_struct(pk), cos.to(dev), sin.to(dev), seqlens.to(dev), xd, out, ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    return out, ref, pk, kc_o, vc_o


@pytest.mark.parametrize("shape,B,ctx", [(O.TINY, 16, 37), (O.TINY_GQA, 32, 50), (O.TINY, 9, 20), (O.TINY_GQA, 128, 140)])
def test_decode_layer_tiles_match_oracle(dev, shape, B, ctx):
    out, ref, pk, kc_o, vc_o = _layer_case(dev, shape, B, ctx, S_max=ctx + 8)
    assert rel_linf(pk["k_cache"], kc_o) <= TOL
    assert rel_linf(pk["v_cache"], vc_o) <= TOL
    assert rel_linf(out, ref) <= TOL


GQA8_DH128 = O.Shape(d=512, H=8, Hk=1, Dh=128, I=512, Rq=96, Rk=32, Rv=32, Ro=96, Rg=96, Ru=96, Rd=96, vocab=300, n_layers=2)
GQA4_DH128 = O.Shape(d=512, H=8, Hk=2, Dh=128, I=512, Rq=96, Rk=64, Rv=64, Ro=96, Rg=96, Ru=96, Rd=96, vocab=300, n_layers=2)


@pytest.mark.parametrize("shape,B,ctx", [(GQA8_DH128, 9, 700), (GQA4_DH128, 10, 391), (O.TINY_GQA, 12, 333),
                                         (GQA8_DH128, 5, 31)])
def test_decode_layer_tiles_grouped_query_heads_long_context(dev, shape, B, ctx):
    """4 and 8 query heads per kv head (the tensor-core decode attention): several key splits per
    sequence, several 32-key blocks per warp, ragged lengths, a last block that is not full."""
    out, ref, pk, kc_o, vc_o = _layer_case(dev, shape, B, ctx, S_max=ctx + 12)
    err = rel_linf(out, ref)
    print(f"H/Hk={shape.H // shape.Hk} Dh={shape.Dh} B={B} ctx={ctx}: rel_linf {err:.3e}")
    assert err <= 2e-2
    assert rel_linf(pk["k_cache"], kc_o) <= 2e-2 and rel_linf(pk["v_cache"], vc_o) <= 2e-2


def test_decode_layer_tiles_ragged_ranks(dev):
    # sizes that are multiples of 8 but of nothing larger: ragged last k-blocks and row tiles
    shape = O.Shape(d=264, H=4, Hk=2, Dh=64, I=520, Rq=88, Rk=40, Rv=56, Ro=72, Rg=104, Ru=104, Rd=80,
                    vocab=200, n_layers=1)
    out, ref, pk, kc_o, vc_o = _layer_case(dev, shape, 24, 21, S_max=32)
    assert rel_linf(pk["k_cache"], kc_o) <= TOL
    assert rel_linf(out, ref) <= TOL


@pytest.mark.parametrize("B", [16, 32])
def test_decode_layer_tiles_7b_shape(dev, B):
    # one Llama-2-7B-shaped layer, ranks 1024 / 1488, 512 cached positions
    out, ref, pk, kc_o, vc_o = _layer_case(dev, O.LLAMA7B_SVD50, B, ctx=512, S_max=516, seed=2)
    assert rel_linf(pk["k_cache"][:, 500:], kc_o[:, 500:]) <= TOL
    assert rel_linf(pk["v_cache"][:, 500:], vc_o[:, 500:]) <= TOL
    assert rel_linf(out, ref) <= TOL


def _engine(dev, *, n_layers, batch, ctx, share_pairs=False, max_new=16):
    import dataclasses

    from flashsvd_b200 import synthetic

    shape = dataclasses.replace(synthetic.LLAMA7B_SVD50, n_layers=n_layers)
    eng = synthetic.make_engine(shape, device=dev, dtype=torch.bfloat16, batch=batch, ctx=ctx, max_new=max_new, seed=0,
                                share_pairs=share_pairs)
    return eng, shape


@pytest.mark.parametrize("batch,ctx,share", [(16, 512, False), (32, 2048, True)])
def test_model_tiles_teacher_forced(dev, batch, ctx, share):
    """Whole-model steps (embed, layers, final norm, lm_head, argmax; one CUDA graph launch per
    step) at the 7B width, 2 layers: logits of every step against the CPU oracle stepped on the GPU's
    tokens.  (32, 2048, shared bases) is configuration 2's batch, context and factor layout."""
    from oracle import check as OC

    eng, shape = _engine(dev, n_layers=2, batch=batch, ctx=ctx, share_pairs=share)
    assert eng.num_stages > 20          # launches per step here, not stages of one kernel
    res = OC.teacher_forced(eng, shape, 3)
    assert eng.status() == 0
    eng.close()
    print(f"B={batch} ctx={ctx}: logits rel_linf {[f'{v:.3e}' for v in res['rel_linf']]}, tokens equal "
          f"{res['n_equal']}/{res['n_tokens']}")
    assert max(res["rel_linf"]) <= 4e-2   # two layers + head; the per-layer bound is 2e-2
    assert res["tokens_explained"]


def test_engine_group_runs_a_batch_wider_than_one_launch(dev):
    """fp32 (and int4) factors have no tiled path; a batch wider than their single launch (4 / 8
    sequences) runs as a group of engines over the same factors.  fp32, 6 sequences = 4 + 2: greedy
    tokens identical to the oracle's."""
    from flashsvd_b200 import engine, packing

    shape, dtype, B, L, n_new = O.TINY, torch.float32, 6, 5, 6
    w = O.make_model_weights(shape, seed=3, dtype=dtype)
    layers = [packing.pack_layer(lw, device=dev, dtype=dtype) for lw in w["layers"]]
    grp = engine.EngineGroup(batch_size=B, width=4, layers=layers, embed=w["embed"].to(dev), final_norm=w["norm"].to(dev),
                             lm_head=w["lm_head"].to(dev), num_heads=shape.H, num_kv_heads=shape.Hk, head_dim=shape.Dh,
                             max_cache_len=L + n_new + 4, rope_theta=shape.theta, eps=shape.eps, max_steps=L + n_new + 8)
    assert [e.B for e in grp.engines] == [4, 2]
    prompt = torch.randint(0, shape.vocab, (B, L), generator=torch.Generator().manual_seed(1))
    grp.prefill(prompt)
    grp.step(n_new - 1)
    torch.cuda.synchronize()
    assert grp.status() == 0
    got = grp.last_tokens(n_new).t().cpu().long()
    ref, _, _ = O.greedy_decode(shape, w, prompt, n_new)
    assert torch.equal(got, ref.long())
    grp.close()


def test_tiles_flag_a_full_cache_and_leave_it_untouched(dev):
    """A token at position S_max on the tiled path: the key / value are not stored and the status
    word says so (FSVD_ERR_CACHE_FULL -> IndexError), as on the single-launch path."""
    from flashsvd_b200 import ops, packing

    shape, dtype, B, S_max = O.TINY, torch.bfloat16, 12, 16
    gen = torch.Generator().manual_seed(4)
    w = O.make_layer_weights(shape, gen, dtype)
    pk = packing.pack_layer(w, device=dev, dtype=dtype)
    kc = torch.randn(B, S_max, shape.Hk, shape.Dh, generator=gen).to(dtype).to(dev)
    vc = torch.randn(B, S_max, shape.Hk, shape.Dh, generator=gen).to(dtype).to(dev)
    pk["k_cache"], pk["v_cache"] = kc.clone(), vc.clone()
    seqlens = torch.full((B,), S_max - 1, dtype=torch.int32)
    seqlens[3] = S_max                      # one sequence is already full
    dims = ops.make_dims(dtype=dtype, B=B, d=shape.d, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, I=shape.I, Rq=shape.Rq,
                         Rk=shape.Rk, Rv=shape.Rv, Ro=shape.Ro, Rg=shape.Rg, Ru=shape.Ru, Rd=shape.Rd, S_max=S_max,
                         eps=shape.eps)
    ws = ops.make_workspace(dims, dev)
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    x = torch.randn(B, shape.d, generator=gen).to(dtype).to(dev)
    out = torch.empty_like(x)
    ops.decode_layer(dims, ops.make_layer_struct(pk), cos.to(dev), sin.to(dev), seqlens.to(dev), x, out, ws)
    torch.cuda.synchronize()
    assert ws.raw_status() == 4
    with pytest.raises(IndexError):
        ws.status()
    assert torch.equal(pk["k_cache"][3], kc[3]) and torch.equal(pk["v_cache"][3], vc[3])   # nothing written for it
    assert not torch.equal(pk["k_cache"][0], kc[0])                                         # the others appended
    ws.clear_status()
    assert ws.status() == 0


def test_small_bf16_batches_take_the_faster_path_and_both_agree(dev):
    """bf16 batches of 5..8 run on the tiled path through fsvd_decode_layer (it is faster there);
    the single-launch kernel is still behind the per-op entry points.  Both against the oracle at
    batch 6, and the launch counts show which path ran."""
    from flashsvd_b200 import ops

    n0 = ops.launch_count()
    out, ref, pk, kc_o, vc_o = _layer_case(dev, O.TINY_GQA, 6, 30, S_max=40, seed=9)
    assert ops.launch_count() - n0 > 5          # several launches: the tiled path
    assert rel_linf(out, ref) <= TOL and rel_linf(pk["k_cache"], kc_o) <= TOL
    n0 = ops.launch_count()
    out4, ref4, *_ = _layer_case(dev, O.TINY_GQA, 4, 30, S_max=40, seed=9)
    assert ops.launch_count() - n0 == 1         # one cooperative launch: the interpreter
    assert rel_linf(out4, ref4) <= TOL
