"""The reference's kernel-level Python entry points, served by the CUDA library (GPU)."""
import pytest
import torch

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


def rel_linf(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 2e-5)])
def test_mlp_dual_split_pcat_s_wrapper(dtype, tol):
    # operands in the reference's layout: GateU/UpU [R, D], DownV [D, R], DownU [R, H]
    from flashsvd_b200 import runtime as R

    dev = torch.device("cuda:0")
    shape = O.TINY
    gen = torch.Generator().manual_seed(3)
    w = O.make_layer_weights(shape, gen, dtype)
    B = 2
    pcat = torch.randn(B, 1, shape.Ru + shape.Rg, generator=gen).to(dtype)
    b2 = torch.randn(shape.d, generator=gen).to(dtype)
    args = [pcat, w["gate_u"].t().contiguous(), w["up_u"].t().contiguous(), w["down_v"].t().contiguous(),
            w["down_u"].t().contiguous()]
    y = R.flashsvd_mlp_dual_split_triton_pcat_s(*[a.to(dev) for a in args], BT=16, num_warps=4)
    ref = O.mlp_from_pcat(pcat[:, 0], w)
    assert y.shape == (B, 1, shape.d)
    assert rel_linf(y[:, 0], ref) <= tol
    yb = R.flashsvd_mlp_dual_split_triton_pcat_s(*[a.to(dev) for a in args], b2.to(dev))
    assert rel_linf(yb[:, 0], (ref.float() + b2.float())) <= tol
    with pytest.raises(ValueError, match="PCat must be"):
        R.flashsvd_mlp_dual_split_triton_pcat_s(pcat[:, 0].to(dev), *[a.to(dev) for a in args[1:]])
    with pytest.raises(ValueError, match="DownV must be"):
        R.flashsvd_mlp_dual_split_triton_pcat_s(args[0].to(dev), args[1].to(dev), args[2].to(dev),
                                                args[3].t().contiguous().to(dev), args[4].to(dev))


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 2e-5)])
def test_reconstruct_qkv_prepacked_wrapper(dtype, tol):
    from flashsvd_b200 import runtime as R

    dev = torch.device("cuda:0")
    shape = O.TINY_GQA
    gen = torch.Generator().manual_seed(4)
    w = O.make_layer_weights(shape, gen, dtype)
    H, Hk, Dh = shape.H, shape.Hk, shape.Dh
    # per-head bases [H, R, Dh] as the reference modules expose them, then prepacked
    Vq = w["q_u"].reshape(H, Dh, shape.Rq).permute(0, 2, 1).contiguous().to(dev)
    Vk = w["k_u"].reshape(Hk, Dh, shape.Rk).permute(0, 2, 1).contiguous().to(dev)
    Vv = w["v_u"].reshape(Hk, Dh, shape.Rv).permute(0, 2, 1).contiguous().to(dev)
    Vq_f, Vk_f, Vv_f = R.pack_qkv_shared_bases(Vq, Vk, Vv)
    assert Vq_f.shape == (shape.Rq, H * Dh) and torch.equal(Vq_f, w["q_u"].t().contiguous().to(dev))
    B = 2
    Pq = torch.randn(B, shape.Rq, generator=gen).to(dtype)
    Pk = torch.randn(B, shape.Rk, generator=gen).to(dtype)
    Pv = torch.randn(B, shape.Rv, generator=gen).to(dtype)
    q, k, v = R.reconstruct_qkv_token_shared_prepacked(Pq.to(dev), Pk.to(dev), Pv.to(dev), Vq_f, Vk_f, Vv_f,
                                                       H=H, Hk=Hk, Dh=Dh)
    lin = torch.nn.functional.linear
    assert q.shape == (B, H, Dh) and k.shape == (B, Hk, Dh) and v.shape == (B, Hk, Dh)
    assert rel_linf(q.reshape(B, -1), lin(Pq.float(), w["q_u"].float())) <= tol
    assert rel_linf(k.reshape(B, -1), lin(Pk.float(), w["k_u"].float())) <= tol
    assert rel_linf(v.reshape(B, -1), lin(Pv.float(), w["v_u"].float())) <= tol


class _Tok:
    eos_token_id = None
    pad_token_id = 0

    def __call__(self, prompt, return_tensors="pt", add_special_tokens=False):
        return {"input_ids": torch.tensor([[int(t) for t in prompt.split()]], dtype=torch.long)}

    def decode(self, ids, skip_special_tokens=False):
        return " ".join(str(int(i)) for i in ids)


def test_generate_text_matches_oracle_greedy():
    from flashsvd_b200 import engine, packing
    from flashsvd_b200 import runtime as R

    dev = torch.device("cuda:0")
    shape, dtype = O.TINY, torch.float32
    w = O.make_model_weights(shape, seed=1, dtype=dtype)
    layers = [packing.pack_layer(lw, device=dev, dtype=dtype) for lw in w["layers"]]
    prompt = torch.randint(0, shape.vocab, (1, 6), generator=torch.Generator().manual_seed(2))
    eng = engine.DecodeEngine(layers=layers, embed=w["embed"].to(dev), final_norm=w["norm"].to(dev),
                              lm_head=w["lm_head"].to(dev), num_heads=shape.H, num_kv_heads=shape.Hk,
                              head_dim=shape.Dh, batch_size=1, max_cache_len=32, rope_theta=shape.theta,
                              eps=shape.eps, max_steps=64)
    res = R.generate_text(eng, _Tok(), prompt=" ".join(str(int(t)) for t in prompt[0]), max_new_tokens=10)
    ref, _, _ = O.greedy_decode(shape, w, prompt, 10)
    assert res["prompt_token_count"] == 6 and res["generated_token_count"] == 10
    assert res["completion_ids"] == ref[0].tolist()
    assert res["output_ids"] == prompt[0].tolist() + ref[0].tolist()
    assert res["completion_text"] == " ".join(str(t) for t in res["completion_ids"])
    # second call reuses the engine from a clean state
    res2 = R.generate_text(eng, _Tok(), prompt=" ".join(str(int(t)) for t in prompt[0]), max_new_tokens=4)
    assert res2["completion_ids"] == ref[0].tolist()[:4]
    with pytest.raises(IndexError):
        R.generate_text(eng, _Tok(), prompt="1 2 3", max_new_tokens=40)
    eng.close()
