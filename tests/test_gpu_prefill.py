"""GPU parity tests of the chunked prompt pass (rows_are_positions of fsvd_dims): the rows of one
launch are consecutive positions of one sequence, share its cache and attend causally.

Oracle: the token-by-token loop of the CPU restatement (utils/evaluator.py:39-82 restated in
oracle.lowrank_llama.decode_step).  fp32: logits within 2e-5 and identical greedy tokens; bf16:
logits within 4e-2 over two layers and the head (2e-2 per layer)."""
import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


def rel_linf(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from flashsvd_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")


def _engine(dev, shape, dtype, w, S_max, chunk):
    from flashsvd_b200 import engine, packing

    layers = [packing.pack_layer(lw, device=dev, dtype=dtype) for lw in w["layers"]]
    return engine.DecodeEngine(layers=layers, embed=w["embed"].to(dev), final_norm=w["norm"].to(dev),
                               lm_head=w["lm_head"].to(dev), num_heads=shape.H, num_kv_heads=shape.Hk,
                               head_dim=shape.Dh, batch_size=1, max_cache_len=S_max, rope_theta=shape.theta,
                               eps=shape.eps, max_steps=S_max + 8, prefill_chunk=chunk)


@pytest.mark.parametrize("dtype,shape,L", [(torch.float32, O.TINY, 23), (torch.float32, O.TINY_GQA, 9),
                                           (torch.bfloat16, O.TINY, 37), (torch.bfloat16, O.TINY_GQA, 17)])
def test_chunked_prompt_pass_matches_oracle(dev, dtype, shape, L):
    n_new, S_max = 6, L + 12
    w = O.make_model_weights(shape, seed=4, dtype=dtype)
    prompt = torch.randint(0, shape.vocab, (1, L), generator=torch.Generator().manual_seed(L))
    toks_ref, logits_ref, st = O.greedy_decode(shape, w, prompt, n_new, S_max=S_max)
    eng = _engine(dev, shape, dtype, w, S_max, None)
    assert eng.prefill_chunk == (4 if dtype == torch.float32 else 8)
    eng.prefill(prompt)
    torch.cuda.synchronize()
    assert eng.status() == 0
    assert int(eng.seqlens[0]) == L
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    assert rel_linf(eng.logits, logits_ref[0]) <= tol
    # the cache rows the chunks wrote, against the oracle's cache (layer 0 and the last layer)
    for li in (0, shape.n_layers - 1):
        assert rel_linf(eng.key_cache[li][:, :L], st.k[li][:, :L]) <= tol
        assert rel_linf(eng.value_cache[li][:, :L], st.v[li][:, :L]) <= tol
    if dtype == torch.float32:
        eng.step(n_new - 1)
        torch.cuda.synchronize()
        # the first generated token is in `tokens` after the prompt pass; the log holds the steps
        log = eng.token_log[: eng.step_counter.item()].cpu().long().flatten()
        assert torch.equal(log[-n_new:], toks_ref[0].long())
    eng.close()


def test_chunked_and_token_by_token_agree(dev):
    # the same engine class with chunks of 1: identical caches and logits in fp32
    shape, dtype, L = O.TINY, torch.float32, 21
    w = O.make_model_weights(shape, seed=6, dtype=dtype)
    prompt = torch.randint(0, shape.vocab, (1, L), generator=torch.Generator().manual_seed(2))
    outs = []
    for chunk in (1, 4, 3):
        eng = _engine(dev, shape, dtype, w, L + 8, chunk)
        eng.prefill(prompt)
        torch.cuda.synchronize()
        assert eng.status() == 0
        outs.append((eng.logits.clone().cpu(), eng.key_cache[1][:, :L].clone().cpu(), int(eng.tokens[0])))
        eng.close()
    for lg, kc, tk in outs[1:]:
        assert rel_linf(lg, outs[0][0]) <= 2e-5
        assert rel_linf(kc, outs[0][1]) <= 2e-5
        assert tk == outs[0][2]


def test_layer_rows_as_positions_matches_oracle(dev):
    # one fsvd_decode_layer call over 4 consecutive positions against 4 oracle steps
    from flashsvd_b200 import ops, packing

    shape, dtype, C, ctx, S_max = O.TINY_GQA, torch.float32, 4, 11, 32
    gen = torch.Generator().manual_seed(8)
    w = O.make_layer_weights(shape, gen, dtype)
    x = torch.randn(C, shape.d, generator=gen)
    kc = torch.zeros(1, S_max, shape.Hk, shape.Dh)
    vc = torch.zeros_like(kc)
    kc[:, :ctx] = torch.randn(1, ctx, shape.Hk, shape.Dh, generator=gen)
    vc[:, :ctx] = torch.randn(1, ctx, shape.Hk, shape.Dh, generator=gen)
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    kco, vco = kc.clone(), vc.clone()
    ref = torch.cat([O.decode_layer(shape, w, x[i:i + 1], kco, vco, torch.tensor([ctx + i], dtype=torch.int32), cos, sin)
                     for i in range(C)])
    pk = packing.pack_layer(w, device=dev, dtype=dtype)
    pk["k_cache"], pk["v_cache"] = kc.to(dev), vc.to(dev)
    dims = ops.make_dims(dtype=dtype, B=C, d=shape.d, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, I=shape.I, Rq=shape.Rq,
                         Rk=shape.Rk, Rv=shape.Rv, Ro=shape.Ro, Rg=shape.Rg, Ru=shape.Ru, Rd=shape.Rd, S_max=S_max,
                         eps=shape.eps, rows_are_positions=1)
    ws = ops.make_workspace(dims, dev)
    out = torch.empty(C, shape.d, dtype=dtype, device=dev)
    seq = (torch.arange(C, dtype=torch.int32) + ctx).to(dev)
    ops.decode_layer(dims, ops.make_layer_struct(pk), cos.to(dev), sin.to(dev), seq, x.to(dev), out, ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert rel_linf(out, ref) <= 2e-5
    assert rel_linf(pk["k_cache"], kco) <= 2e-5 and rel_linf(pk["v_cache"], vco) <= 2e-5


DH128 = O.Shape(d=256, H=2, Hk=2, Dh=128, I=512, Rq=64, Rk=64, Rv=64, Ro=64, Rg=96, Ru=96, Rd=96, vocab=300, n_layers=2)
DH128_GQA = O.Shape(d=512, H=8, Hk=1, Dh=128, I=512, Rq=96, Rk=32, Rv=32, Ro=96, Rg=96, Ru=96, Rd=96, vocab=300, n_layers=2)


@pytest.mark.parametrize("shape,L", [(O.TINY, 300), (O.TINY_GQA, 131), (DH128, 150), (DH128_GQA, 140)])
def test_tiled_prompt_pass_matches_oracle(dev, shape, L):
    """Prompts longer than 128 tokens (bf16, one sequence): 128 positions per pass through the tiled
    tensor-core GEMMs (rows_are_positions with B = 128) and the tensor-core causal attention
    (head_dim 64 and 128, 1 / 4 / 8 query heads per kv head), then smaller passes, then token by
    token; caches and the first logits against the oracle's token-by-token loop."""
    dtype, n_new, S_max = torch.bfloat16, 2, L + 12
    w = O.make_model_weights(shape, seed=7, dtype=dtype)
    prompt = torch.randint(0, shape.vocab, (1, L), generator=torch.Generator().manual_seed(L))
    toks_ref, logits_ref, st = O.greedy_decode(shape, w, prompt, n_new, S_max=S_max)
    eng = _engine(dev, shape, dtype, w, S_max, None)
    assert eng.prefill_tile == 128
    eng.prefill(prompt)
    torch.cuda.synchronize()
    assert eng.status() == 0
    assert 128 in eng._chunks          # the tiled pass ran
    assert int(eng.seqlens[0]) == L
    assert rel_linf(eng.logits, logits_ref[0]) <= 4e-2
    for li in (0, shape.n_layers - 1):
        assert rel_linf(eng.key_cache[li][:, :L], st.k[li][:, :L]) <= 4e-2
        assert rel_linf(eng.value_cache[li][:, :L], st.v[li][:, :L]) <= 4e-2
    eng.close()
