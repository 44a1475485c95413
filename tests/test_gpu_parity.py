"""GPU parity tests: the CUDA path, called through the C ABI (ctypes), against the CPU oracle on
the same seeded inputs.  Tolerances: fp32 storage -> 2e-5 relative (summation order only);
bf16 storage with fp32 accumulation -> per-layer max relative error 2e-2 (rel_linf =
max|y_ref - y| / max|y_ref|, benchmark/decode/check_flashsvd_decode_correctness.py:183-187);
greedy token ids identical in fp32."""
import numpy as np
import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def rel_linf(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from flashsvd_b200 import _lib

    _lib.load()  # fails loudly if the CUDA library is missing
    return torch.device("cuda:0")


def _dims(ops, shape, dtype, B, S_max, **kw):
    return ops.make_dims(dtype=dtype, B=B, d=shape.d, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, I=shape.I, Rq=shape.Rq,
                         Rk=shape.Rk, Rv=shape.Rv, Ro=shape.Ro, Rg=shape.Rg, Ru=shape.Ru, Rd=shape.Rd,
                         S_max=S_max, eps=shape.eps, **kw)


def _layer_case(dev, shape, dtype, B, ctx, S_max, seed=0):
    from flashsvd_b200 import ops, packing

    gen = torch.Generator().manual_seed(seed)
    w = O.make_layer_weights(shape, gen, dtype)
    x = torch.randn(B, shape.d, generator=gen).to(dtype)
    kc = torch.zeros(B, S_max, shape.Hk, shape.Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    if ctx:
        kc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen).to(dtype)
        vc[:, :ctx] = torch.randn(B, ctx, shape.Hk, shape.Dh, generator=gen).to(dtype)
    seqlens = torch.full((B,), ctx, dtype=torch.int32)
    if B > 1 and ctx > 3:
        seqlens[1] = ctx - 3  # ragged batch
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    kc_o, vc_o = kc.clone(), vc.clone()
    ref = O.decode_layer(shape, w, x, kc_o, vc_o, seqlens, cos, sin)
    pk = packing.pack_layer(w, device=dev, dtype=dtype)
    pk["k_cache"], pk["v_cache"] = kc.to(dev), vc.to(dev)
    dims = _dims(ops, shape, dtype, B, S_max)
    ws = ops.make_workspace(dims, dev)
    out = torch.empty(B, shape.d, dtype=dtype, device=dev)
    ops.decode_layer(dims, ops.make_layer_struct(pk), cos.to(dev), sin.to(dev), seqlens.to(dev), x.to(dev), out, ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    return out, ref, pk, kc_o, vc_o


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,B,ctx", [(O.TINY, 1, 37), (O.TINY, 2, 37), (O.TINY_GQA, 2, 50), (O.TINY, 1, 0),
                                         (O.TINY, 3, 59)])
def test_decode_layer_matches_oracle(dev, dtype, shape, B, ctx):
    out, ref, pk, kc_o, vc_o = _layer_case(dev, shape, dtype, B, ctx, S_max=64)
    assert rel_linf(out, ref) <= TOL[dtype]
    assert rel_linf(pk["k_cache"], kc_o) <= TOL[dtype]
    assert rel_linf(pk["v_cache"], vc_o) <= TOL[dtype]


def test_decode_layer_last_cache_slot(dev):
    # the new token lands in the last position of the cache
    out, ref, pk, kc_o, _ = _layer_case(dev, O.TINY, torch.float32, 1, ctx=63, S_max=64)
    assert rel_linf(out, ref) <= 2e-5
    assert rel_linf(pk["k_cache"][:, 63], kc_o[:, 63]) <= 2e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_decode_layer_7b_shape(dev, dtype):
    # configuration 0: one Llama-2-7B-shaped layer, ranks 1024 / 1488, 512 cached positions
    out, ref, pk, kc_o, vc_o = _layer_case(dev, O.LLAMA7B_SVD50, dtype, 1, ctx=512, S_max=516)
    assert rel_linf(out, ref) <= TOL[dtype]
    assert rel_linf(pk["k_cache"][:, 512], kc_o[:, 512]) <= TOL[dtype]
    assert rel_linf(pk["v_cache"][:, 512], vc_o[:, 512]) <= TOL[dtype]


def test_ragged_shapes(dev):
    # ranks and sizes that are multiples of 8 but of nothing larger: ragged last blocks and row groups
    shape = O.Shape(d=264, H=4, Hk=2, Dh=64, I=520, Rq=88, Rk=40, Rv=56, Ro=72, Rg=104, Ru=104, Rd=80,
                    vocab=200, n_layers=1)
    for dtype in (torch.float32, torch.bfloat16):
        out, ref, *_ = _layer_case(dev, shape, dtype, 2, ctx=21, S_max=32)
        assert rel_linf(out, ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_op_entry_points(dev, dtype):
    from flashsvd_b200 import ops

    shape, B, S_max, ctx = O.TINY_GQA, 2, 48, 30
    gen = torch.Generator().manual_seed(5)
    w = O.make_layer_weights(shape, gen, dtype)
    d = {k: v.to(dev) for k, v in w.items()}
    dims = _dims(ops, shape, dtype, B, S_max)
    ws = ops.make_workspace(dims, dev)
    tol = TOL[dtype]
    # low-rank projection with and without residual
    a = torch.randn(B, shape.H * shape.Dh, generator=gen).to(dtype)
    res = torch.randn(B, shape.d, generator=gen).to(dtype)
    y = ops.lowrank_proj(a.to(dev), d["o_v"], d["o_u"], ws)
    assert rel_linf(y, O.lowrank(a, w["o_v"], w["o_u"])) <= tol
    y = ops.lowrank_proj(a.to(dev), d["o_v"], d["o_u"], ws, residual=res.to(dev))
    assert rel_linf(y, res + O.lowrank(a, w["o_v"], w["o_u"])) <= tol
    # MLP from PCat = [p_up | p_gate] and from the hidden state with RMSNorm
    x = torch.randn(B, shape.d, generator=gen).to(dtype)
    pcat = torch.cat([torch.nn.functional.linear(x, w["up_v"]), torch.nn.functional.linear(x, w["gate_v"])], 1)
    y = ops.mlp_swiglu_decode(pcat.to(dev), d["gate_u"], d["up_u"], d["down_v"], d["down_u"], ws)
    assert rel_linf(y, O.mlp_from_pcat(pcat, w)) <= tol
    upgate = torch.cat([w["up_v"], w["gate_v"]], 0).to(dev).contiguous()
    y = ops.mlp_swiglu_decode(x.to(dev), d["gate_u"], d["up_u"], d["down_v"], d["down_u"], ws, upgate_v=upgate,
                              norm_w=d["ln2"], eps=shape.eps, residual=x.to(dev))
    xn = O.rmsnorm(x, w["ln2"], shape.eps)
    pc = torch.cat([torch.nn.functional.linear(xn, w["up_v"]), torch.nn.functional.linear(xn, w["gate_v"])], 1)
    assert rel_linf(y, x + O.mlp_from_pcat(pc, w)) <= tol
    # q/k/v with rotary and cache append, then attention
    kc = torch.randn(B, S_max, shape.Hk, shape.Dh, generator=gen).to(dtype)
    vc = torch.randn(B, S_max, shape.Hk, shape.Dh, generator=gen).to(dtype)
    seq = torch.tensor([ctx, ctx - 7], dtype=torch.int32)
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    kcd, vcd = kc.to(dev), vc.to(dev)
    qkv_v = torch.cat([w["q_v"], w["k_v"], w["v_v"]], 0).to(dev).contiguous()
    q = ops.qkv_rope_append(x.to(dev), qkv_v, d["q_u"], d["k_u"], d["v_u"], cos.to(dev), sin.to(dev), kcd, vcd,
                            seq.to(dev), ws, num_heads=shape.H, num_kv_heads=shape.Hk, head_dim=shape.Dh,
                            ranks=(shape.Rq, shape.Rk, shape.Rv), norm_w=d["ln1"], eps=shape.eps)
    out = ops.flash_decode(q, kcd, vcd, seq.to(dev), ws, seqlen_add=1)
    torch.cuda.synchronize()
    assert ws.status() == 0
    tr = {}
    kco, vco = kc.clone(), vc.clone()
    O.decode_layer(shape, w, x, kco, vco, seq, cos, sin, trace=tr)
    assert rel_linf(q, tr["q"]) <= tol
    assert rel_linf(kcd, kco) <= tol and rel_linf(vcd, vco) <= tol
    assert rel_linf(out.reshape(B, -1), tr["attn"]) <= tol


def _greedy(dev, shape, dtype, prompt, n_new, seed=0):
    from flashsvd_b200 import engine, packing

    w = O.make_model_weights(shape, seed=seed, dtype=dtype)
    layers = [packing.pack_layer(lw, device=dev, dtype=dtype) for lw in w["layers"]]
    B, L = prompt.shape
    eng = engine.DecodeEngine(layers=layers, embed=w["embed"].to(dev), final_norm=w["norm"].to(dev),
                              lm_head=w["lm_head"].to(dev), num_heads=shape.H, num_kv_heads=shape.Hk,
                              head_dim=shape.Dh, batch_size=B, max_cache_len=L + n_new + 4,
                              rope_theta=shape.theta, eps=shape.eps, max_steps=L + n_new + 8)
    eng.prefill(prompt)
    torch.cuda.synchronize()
    logits0 = eng.logits.clone().cpu()
    eng.step(n_new - 1)
    torch.cuda.synchronize()
    # the log has one row per single-token launch (a single sequence's prompt goes in chunks, which
    # are not logged): the last n_new rows are the generated tokens
    toks = eng.last_tokens(n_new).t().cpu().long()
    assert eng.status() == 0
    eng.close()
    return toks, logits0, w


@pytest.mark.parametrize("name,shape", [("tiny", O.TINY), ("gqa", O.TINY_GQA)])
def test_greedy_tokens_match_reference_golden_fp32(dev, golden, name, shape):
    # 8 greedy tokens produced by the reference's own decode loop and cache (tests/golden)
    prompt = torch.from_numpy(golden[f"{name}_f32_prompt"])
    toks, logits0, _ = _greedy(dev, shape, torch.float32, prompt, 8)
    assert np.array_equal(toks.numpy(), golden[f"{name}_f32_tokens"])
    ref = torch.from_numpy(golden[f"{name}_f32_logits0"])
    assert rel_linf(logits0, ref) <= 2e-5


def test_greedy_32_steps_identical_fp32(dev):
    # identical greedy tokens over 32 decode steps in fp32 mode, 4-layer model at reduced width
    shape = O.Shape(d=512, H=8, Hk=8, Dh=64, I=1376, Rq=128, Rk=128, Rv=128, Ro=128, Rg=184, Ru=184, Rd=184,
                    vocab=1000, n_layers=4)
    prompt = torch.randint(0, shape.vocab, (2, 12), generator=torch.Generator().manual_seed(9))
    toks, _, w = _greedy(dev, shape, torch.float32, prompt, 32)
    ref, _, _ = O.greedy_decode(shape, w, prompt, 32)
    assert torch.equal(toks, ref.long())


def test_greedy_bf16_logits_within_tolerance(dev, golden):
    prompt = torch.from_numpy(golden["tiny_bf16_prompt"])
    toks, logits0, _ = _greedy(dev, O.TINY, torch.bfloat16, prompt, 8)
    ref = torch.from_numpy(golden["tiny_bf16_logits0"])
    assert rel_linf(logits0, ref) <= 4e-2  # two layers + head; per-layer bound is 2e-2
    assert np.array_equal(toks.numpy(), golden["tiny_bf16_tokens"])


def test_full_size_properties(dev):
    """Size-independent properties at the 7B shape: scaling the input by 2 scales a low-rank
    projection by exactly 2, two runs are bitwise identical, attention outputs stay inside the
    range of the cached values."""
    from flashsvd_b200 import ops

    shape, dtype = O.LLAMA7B_SVD50, torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    v = (torch.randn(shape.Rd, shape.I, device=dev, generator=g) / shape.I ** 0.5).to(dtype)
    u = (torch.randn(shape.d, shape.Rd, device=dev, generator=g) / shape.Rd ** 0.5).to(dtype)
    x = torch.randn(1, shape.I, device=dev, generator=g).to(dtype)
    dims = ops.make_dims(dtype=dtype, B=1, d=shape.d, H=shape.H, Hk=shape.Hk, Dh=shape.Dh, I=shape.I, Ro=shape.Rd,
                         Rd=shape.Rd, S_max=1024)
    ws = ops.make_workspace(dims, dev)
    y1 = ops.lowrank_proj(x, v, u, ws).clone()
    y2 = ops.lowrank_proj(x, v, u, ws).clone()
    y3 = ops.lowrank_proj(x * 2, v, u, ws).clone()
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert torch.equal(y3.float(), y1.float() * 2)
    ref = torch.nn.functional.linear(torch.nn.functional.linear(x.float(), v.float()).to(dtype).float(), u.float())
    assert rel_linf(y1, ref) <= 2e-2
    S = 1024
    q = torch.randn(1, shape.H, shape.Dh, device=dev, generator=g).to(dtype)
    kc = torch.randn(1, S, shape.Hk, shape.Dh, device=dev, generator=g).to(dtype)
    vc = torch.randn(1, S, shape.Hk, shape.Dh, device=dev, generator=g).to(dtype)
    seq = torch.tensor([S], dtype=torch.int32, device=dev)
    o1 = ops.flash_decode(q, kc, vc, seq, ws).clone()
    o2 = ops.flash_decode(q, kc, vc, seq, ws).clone()
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)
    assert float(o1.float().abs().max()) <= float(vc.float().abs().max())
    refa = torch.stack([O.attend(q[0].cpu().float(), kc[0].cpu().float(), vc[0].cpu().float())])
    assert rel_linf(o1, refa) <= 2e-2
    assert ws.status() == 0


def test_argument_errors_raise_before_launch(dev):
    from flashsvd_b200 import ops

    dims = ops.make_dims(dtype=torch.float32, B=1, d=64, Ro=16)
    ws = ops.make_workspace(dims, dev)
    x = torch.zeros(1, 64, device=dev)
    with pytest.raises(ValueError):
        ops.lowrank_proj(x, torch.zeros(16, 32, device=dev), torch.zeros(64, 16, device=dev), ws)  # shape mismatch
    with pytest.raises(ValueError):
        ops.lowrank_proj(x, torch.zeros(12, 64, device=dev), torch.zeros(64, 12, device=dev), ws)  # rank not % 8
    with pytest.raises(ValueError):
        ops.lowrank_proj(x.half(), torch.zeros(16, 64, device=dev).half(), torch.zeros(64, 16, device=dev).half(), ws)
    small = ops.Workspace(torch.zeros(64, dtype=torch.uint8, device=dev), 64)
    with pytest.raises(ValueError):
        ops.lowrank_proj(x, torch.zeros(16, 64, device=dev), torch.zeros(64, 16, device=dev), small)


@pytest.mark.parametrize("dtype,B,d_in,R,d_out", [(torch.bfloat16, 4, 11008, 1488, 4096), (torch.bfloat16, 8, 11008, 1488, 4096),
                                                  (torch.float32, 2, 4096, 1024, 4096), (torch.bfloat16, 2, 4352, 64, 72)])
def test_lowrank_proj_long_input_several_rows(dev, dtype, B, d_in, R, d_out):
    # a long input vector with several batch rows is staged one K segment per CTA
    from flashsvd_b200 import ops

    gen = torch.Generator().manual_seed(B + d_in)
    v_w = (torch.randn(R, d_in, generator=gen) / d_in ** 0.5).to(dtype)
    u_w = (torch.randn(d_out, R, generator=gen) / R ** 0.5).to(dtype)
    x = torch.randn(B, d_in, generator=gen).to(dtype)
    dims = ops.make_dims(dtype=dtype, B=B, d=max(d_in, d_out), I=max(d_in, d_out), Ro=R, Rd=R, Rg=R, Ru=R, Rq=R,
                         Rk=R, Rv=R)
    ws = ops.make_workspace(dims, dev)
    y = ops.lowrank_proj(x.to(dev), v_w.to(dev), u_w.to(dev), ws)
    torch.cuda.synchronize()
    assert ws.status() == 0
    assert rel_linf(y, O.lowrank(x, v_w, u_w)) <= TOL[dtype]


@pytest.mark.parametrize("shape,B,ctx,S_max", [(O.LLAMA7B_SVD50, 4, 300, 304), (O.TINY, 8, 20, 32), (O.TINY_GQA, 7, 9, 16)])
def test_decode_layer_wide_batches(dev, shape, B, ctx, S_max):
    out, ref, pk, kc_o, vc_o = _layer_case(dev, shape, torch.bfloat16, B, ctx, S_max=S_max, seed=3)
    assert rel_linf(out, ref) <= TOL[torch.bfloat16]
    assert rel_linf(pk["k_cache"], kc_o) <= TOL[torch.bfloat16]
    assert rel_linf(pk["v_cache"], vc_o) <= TOL[torch.bfloat16]


@pytest.mark.parametrize("B", [1, 2])
def test_decode_layer_70b_shape(dev, B):
    # one Llama-2-70B-shaped layer: GQA 64/8, ranks 1312 / 224 / 2704 (unequal q/k/v ranks, so three
    # lift stages), 28672-wide MLP input staged one K segment per CTA
    out, ref, pk, kc_o, vc_o = _layer_case(dev, O.LLAMA70B_SVD40, torch.bfloat16, B, ctx=300, S_max=304, seed=5)
    assert rel_linf(out, ref) <= TOL[torch.bfloat16]
    assert rel_linf(pk["k_cache"][:, 300], kc_o[:, 300]) <= TOL[torch.bfloat16]
    assert rel_linf(pk["v_cache"][:, 300], vc_o[:, 300]) <= TOL[torch.bfloat16]
