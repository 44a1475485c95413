"""Module surface (SVD_LlamaAttention / SVD_LlamaMLP) on the GPU against the CPU oracle."""
from types import SimpleNamespace

import pytest
import torch
import torch.nn.functional as F

from oracle import lowrank_llama as O

pytestmark = pytest.mark.gpu


def rel_linf(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def test_rank_formula_and_names():
    from flashsvd_b200 import modules as M

    assert M.svd_rank(4096, 4096, 0.5) == 1024 and M.svd_rank(11008, 4096, 0.5) == 1492
    mlp = M.SVD_LlamaMLP(64, 160, "silu", 0.5)
    assert mlp.gate_v_proj.weight.shape == (mlp.low_rank, 64) and mlp.down_u_proj.weight.shape == (64, mlp.low_rank)
    assert mlp.low_rank % 8 == 0
    cfg = SimpleNamespace(hidden_size=128, num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=64)
    att = M.SVD_LlamaAttention(cfg, 0.5, layer_idx=1)
    assert att.q_u_proj.weight.shape == (128, att.low_rank) and att.k_u_proj.weight.shape[0] == 64
    assert att.num_key_value_groups == 2 and att.head_dim == 64
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mlp(torch.zeros(1, 1, 64))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_mlp_module_decode_and_prompt(dtype, tol):
    from flashsvd_b200 import modules as M

    dev = torch.device("cuda:0")
    shape = O.TINY
    w = O.make_layer_weights(shape, torch.Generator().manual_seed(7), dtype)
    mlp = M.SVD_LlamaMLP(shape.d, shape.I, "silu", 0.5)
    for n in ("gate_v", "gate_u", "up_v", "up_u", "down_v", "down_u"):
        lin = getattr(mlp, n + "_proj")
        lin.weight = torch.nn.Parameter(w[n].clone(), requires_grad=False)
        lin.in_features, lin.out_features = w[n].shape[1], w[n].shape[0]
    mlp = mlp.to(dev)
    x = torch.randn(2, 1, shape.d, generator=torch.Generator().manual_seed(8)).to(dtype)

    def ref(xx):
        g = F.linear(F.linear(xx, w["gate_v"]), w["gate_u"])
        u = F.linear(F.linear(xx, w["up_v"]), w["up_u"])
        return F.linear(F.linear(F.silu(g) * u, w["down_v"]), w["down_u"])

    with torch.inference_mode():
        y = mlp(x.to(dev))
        assert y.shape == (2, 1, shape.d) and rel_linf(y, ref(x)) <= tol
        xl = torch.randn(1, 5, shape.d, generator=torch.Generator().manual_seed(9)).to(dtype)
        assert rel_linf(mlp(xl.to(dev)), ref(xl)) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_attention_module_prompt_then_decode(dtype, tol):
    from flashsvd_b200 import modules as M
    from flashsvd_b200 import runtime as R

    dev = torch.device("cuda:0")
    shape = O.TINY_GQA
    w = O.make_layer_weights(shape, torch.Generator().manual_seed(11), dtype)
    cfg = SimpleNamespace(hidden_size=shape.d, num_attention_heads=shape.H, num_key_value_heads=shape.Hk,
                          head_dim=shape.Dh, num_hidden_layers=1, rope_theta=shape.theta, max_position_embeddings=32)
    att = M.SVD_LlamaAttention(cfg, 0.5, layer_idx=0)
    for n in ("q_v", "q_u", "k_v", "k_u", "v_v", "v_u", "o_v", "o_u"):
        lin = getattr(att, n + "_proj")
        lin.weight = torch.nn.Parameter(w[n].clone(), requires_grad=False)
        lin.in_features, lin.out_features = w[n].shape[1], w[n].shape[0]
    att = att.to(dev)
    B, Lp, S_max = 2, 5, 16
    cache = R.FlashSVDV15DenseKVCache(cfg, max_batch_size=B, max_cache_len=S_max, device=dev, dtype=dtype)
    gen = torch.Generator().manual_seed(12)
    xs = torch.randn(B, Lp + 3, shape.d, generator=gen).to(dtype)

    # oracle: token by token (attention block only: no norm, no residual)
    kc = torch.zeros(B, S_max, shape.Hk, shape.Dh, dtype=dtype)
    vc = torch.zeros_like(kc)
    cos, sin = O.rope_tables(S_max, shape.Dh, shape.theta, dtype)
    ref = []
    for t in range(Lp + 3):
        x = xs[:, t]
        q = F.linear(F.linear(x, w["q_v"]), w["q_u"]).view(B, shape.H, shape.Dh)
        k = F.linear(F.linear(x, w["k_v"]), w["k_u"]).view(B, shape.Hk, shape.Dh)
        v = F.linear(F.linear(x, w["v_v"]), w["v_u"]).view(B, shape.Hk, shape.Dh)
        a = torch.empty(B, shape.H * shape.Dh, dtype=dtype)
        for b in range(B):
            c, s = cos[t].unsqueeze(0), sin[t].unsqueeze(0)
            kc[b, t] = O.rotate_half_apply(k[b], c, s)
            vc[b, t] = v[b]
            a[b] = O.attend(O.rotate_half_apply(q[b], c, s), kc[b, : t + 1], vc[b, : t + 1]).reshape(-1)
        ref.append(O.lowrank(a, w["o_v"], w["o_u"]))
    ref = torch.stack(ref, 1)

    with torch.inference_mode():
        y, wts = att(xs[:, :Lp].to(dev), past_key_values=cache, cache_position=torch.arange(Lp))
        assert wts is None and y.shape == (B, Lp, shape.d)
        assert rel_linf(y, ref[:, :Lp]) <= max(tol, 1e-4)
        assert cache.get_seq_length() == Lp
        for t in range(Lp, Lp + 3):
            y, _ = att(xs[:, t:t + 1].to(dev), past_key_values=cache, cache_position=torch.tensor([t]))
            assert rel_linf(y[:, 0], ref[:, t]) <= tol
        assert cache.get_seq_length() == Lp + 3
        assert rel_linf(cache.key_cache[0][:, :Lp + 3], kc[:, :Lp + 3]) <= tol
