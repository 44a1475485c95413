"""CPU: the reference's local checkpoint formats (utils/model_utils.py:241-522, 525-671, 850-901)
loaded into models made of this package's modules: a basis-sharing export directory (key names,
shards, groups tied to one parameter, the reference's error cases) and wrapped factor pairs."""
import json

import pytest
import torch
import torch.nn as nn

from flashsvd_b200 import checkpoints as CK
from flashsvd_b200 import demo_support as DS
from flashsvd_b200.modules import SVD_LlamaAttention, SVD_LlamaMLP

CFG = dict(hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
           head_dim=16, vocab_size=50, max_position_embeddings=128, rms_norm_eps=1e-5, hidden_act="silu")
R_ATTN, R_MLP = 8, 16


def _export_tensors(seed=0, groups=((0, 1), (2, 3))):
    """Tensors of a basis-sharing export: layers of a group hold the SAME basis for every projection."""
    g = torch.Generator().manual_seed(seed)
    d, I, V = CFG["hidden_size"], CFG["intermediate_size"], CFG["vocab_size"]
    HD, KD = CFG["num_attention_heads"] * CFG["head_dim"], CFG["num_key_value_heads"] * CFG["head_dim"]
    r = lambda *s: torch.randn(*s, generator=g)
    sd = {"model.embed_tokens.weight": r(V, d), "model.norm.weight": r(d), "lm_head.weight": r(V, d)}
    out_dims = {"q": HD, "k": KD, "v": KD, "o": d, "gate": I, "up": I, "down": d}
    in_dims = {"q": d, "k": d, "v": d, "o": HD, "gate": d, "up": d, "down": I}
    rank = {"q": R_ATTN, "k": R_ATTN, "v": R_ATTN, "o": R_ATTN, "gate": R_MLP, "up": R_MLP, "down": R_MLP}
    for grp in groups:
        basis = {n: r(rank[n], in_dims[n]) for n in out_dims}
        for li in grp:
            pre = f"model.layers.{li}"
            sd[f"{pre}.input_layernorm.weight"] = r(d)
            sd[f"{pre}.post_attention_layernorm.weight"] = r(d)
            for n in out_dims:
                holder = "self_attn" if n in ("q", "k", "v", "o") else "mlp"
                sd[f"{pre}.{holder}.{n}_proj.weight"] = r(out_dims[n], rank[n])
                sd[f"{pre}.{holder}.{n}_basis.weight"] = basis[n].clone()
    return sd


def _write_export(tmp_path, sd, *, sharded, groups=((0, 1), (2, 3)), arch="ShareLlamaForCausalLM"):
    cfg = dict(CFG, architectures=[arch], model_type="llama", torch_dtype="float32")
    for name in CK.GROUPS:
        cfg[name] = [list(gp) for gp in groups]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    if not sharded:
        torch.save(sd, tmp_path / "pytorch_model.bin")
        return
    keys = sorted(sd)
    half = len(keys) // 2
    parts = {"pytorch_model-00002-of-00002.bin": keys[half:], "pytorch_model-00001-of-00002.bin": keys[:half]}
    weight_map = {}
    for fname, ks in parts.items():
        torch.save({k: sd[k] for k in ks}, tmp_path / fname)
        weight_map.update({k: fname for k in ks})
    (tmp_path / "pytorch_model.bin.index.json").write_text(json.dumps({"weight_map": weight_map}))


@pytest.mark.parametrize("sharded", [False, True])
def test_basis_sharing_export_loads_with_tied_groups(tmp_path, sharded):
    sd = _export_tensors()
    _write_export(tmp_path, sd, sharded=sharded)
    model, tok = DS.get_model_from_local(str(tmp_path))
    assert tok is None and model.seqlen == CFG["max_position_embeddings"]
    layers = model.model.layers
    assert all(isinstance(l.self_attn, SVD_LlamaAttention) and isinstance(l.mlp, SVD_LlamaMLP) for l in layers)
    # proj -> output-side factor, basis -> input-side factor
    assert torch.equal(layers[2].self_attn.q_u_proj.weight, sd["model.layers.2.self_attn.q_proj.weight"])
    assert torch.equal(layers[2].self_attn.q_v_proj.weight, sd["model.layers.2.self_attn.q_basis.weight"])
    assert torch.equal(layers[1].mlp.down_u_proj.weight, sd["model.layers.1.mlp.down_proj.weight"])
    assert torch.equal(layers[1].mlp.down_v_proj.weight, sd["model.layers.1.mlp.down_basis.weight"])
    assert torch.equal(model.lm_head.weight, sd["lm_head.weight"])
    assert torch.equal(layers[3].input_layernorm.weight, sd["model.layers.3.input_layernorm.weight"])
    # the members of a group hold ONE parameter per shared basis; different groups do not
    for holder, lin in CK.GROUPS.values():
        a, b, c = (getattr(getattr(layers[i], holder), lin).weight for i in (0, 1, 2))
        assert a is b and a is not c
    attn, mlp = layers[0].self_attn, layers[0].mlp
    assert attn.low_rank == R_ATTN and attn.ratio == pytest.approx(2.0 * R_ATTN / 64) and attn.use_lowrank_cache
    assert mlp.ratio == pytest.approx(R_MLP * (64 + 96) / (64 * 96))
    assert attn.q_v_proj.in_features == 64 and attn.q_v_proj.out_features == R_ATTN


def test_basis_sharing_errors_follow_the_reference(tmp_path):
    sd = _export_tensors()
    missing = dict(sd)
    del missing["model.layers.1.mlp.up_basis.weight"], missing["model.layers.3.self_attn.o_proj.weight"]
    _write_export(tmp_path, missing, sharded=False)
    with pytest.raises(KeyError, match="Basis_Sharing load is missing 2 required tensors"):
        DS.get_model_from_local(str(tmp_path))
    broken = dict(sd)
    broken["model.layers.1.self_attn.k_basis.weight"] = broken["model.layers.1.self_attn.k_basis.weight"] + 0.5
    _write_export(tmp_path, broken, sharded=False)
    with pytest.raises(ValueError, match=r"k_groups\[0\] is not actually shared \(layers 0 and 1"):
        DS.get_model_from_local(str(tmp_path))
    ranks = _export_tensors()
    for li in (0, 1):
        ranks[f"model.layers.{li}.self_attn.v_proj.weight"] = torch.randn(32, 4)
        ranks[f"model.layers.{li}.self_attn.v_basis.weight"] = ranks["model.layers.0.self_attn.v_basis.weight"][:4].clone()
    _write_export(tmp_path, ranks, sharded=False)
    with pytest.raises(ValueError, match="must have shared q/k/v rank; got 8/8/4"):
        DS.get_model_from_local(str(tmp_path))


def test_shard_discovery_order_and_errors(tmp_path):
    with pytest.raises(FileNotFoundError, match="Could not find HF PyTorch checkpoint shards"):
        list(CK.iter_weight_shards(tmp_path))
    for n in ("pytorch_model-00002-of-00002.bin", "pytorch_model-00001-of-00002.bin"):
        torch.save({}, tmp_path / n)
    assert [p.name for p in CK.iter_weight_shards(tmp_path)] == ["pytorch_model-00001-of-00002.bin", "pytorch_model-00002-of-00002.bin"]
    (tmp_path / "pytorch_model.bin.index.json").write_text(json.dumps({"weight_map": {"a": "pytorch_model-00002-of-00002.bin",
                                                                                      "b": "gone.bin"}}))
    with pytest.raises(FileNotFoundError, match="Missing shard referenced by index"):
        list(CK.iter_weight_shards(tmp_path))
    (tmp_path / "pytorch_model.bin.index.json").write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(ValueError, match="Invalid HF shard index"):
        list(CK.iter_weight_shards(tmp_path))
    assert CK.basis_sharing_destination("model.layers.7.mlp.gate_basis.weight") == "model.layers.7.mlp.gate_v_proj.weight"
    assert CK.basis_sharing_destination("model.layers.7.self_attn.rotary_emb.inv_freq") is None
    assert not CK.is_basis_sharing_config({"architectures": ["LlamaForCausalLM"]})


class _UV(nn.Module):
    def __init__(self, d_in, d_out, r, dobi=False):
        super().__init__()
        u, v = nn.Linear(r, d_out, bias=False), nn.Linear(d_in, r, bias=False)
        if dobi:
            self.BLinear, self.ALinear = u, v
        else:
            self.u_proj, self.v_proj = u, v


def test_wrapped_factor_pairs_become_native_modules_over_the_same_weights(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(**dict(CFG, num_hidden_layers=2))
    model = LlamaForCausalLM(cfg)
    d, I, HD, KD = 64, 96, 64, 32
    for li, layer in enumerate(model.model.layers):
        dobi = li == 1
        a, m = layer.self_attn, layer.mlp
        a.q_proj, a.k_proj, a.v_proj, a.o_proj = _UV(d, HD, 8, dobi), _UV(d, KD, 8, dobi), _UV(d, KD, 8, dobi), _UV(HD, d, 8, dobi)
        m.gate_proj, m.up_proj, m.down_proj = _UV(d, I, 16, dobi), _UV(d, I, 16, dobi), _UV(I, d, 24, dobi)
    src_u = model.model.layers[1].mlp.down_proj.BLinear.weight
    src_v = model.model.layers[0].self_attn.k_proj.v_proj.weight
    torch.save({"model": model, "tokenizer": "tok"}, tmp_path / "merge.pt")
    loaded, tok = DS.get_model_from_local(str(tmp_path / "merge.pt"))
    assert tok == "tok"
    for li, layer in enumerate(loaded.model.layers):
        assert isinstance(layer.self_attn, SVD_LlamaAttention) and isinstance(layer.mlp, SVD_LlamaMLP)
        assert layer.self_attn.low_rank == 8 and layer.mlp.down_v_proj.out_features == 24
        assert layer.mlp.ratio == pytest.approx(0.5 * 32 * (64 + 96) / (64 * 96))
    assert torch.equal(loaded.model.layers[1].mlp.down_u_proj.weight, src_u)
    assert torch.equal(loaded.model.layers[0].self_attn.k_v_proj.weight, src_v)
    # in memory the conversion shares the parameters instead of copying them
    again = CK.convert_wrapped_factor_pairs(model)
    assert again.model.layers[1].mlp.down_u_proj.weight is src_u
    # a second pass leaves native layers alone
    assert CK.convert_wrapped_factor_pairs(again).model.layers[0].self_attn is again.model.layers[0].self_attn


def test_unrecognised_and_untrusted_local_checkpoints(tmp_path, monkeypatch):
    monkeypatch.delenv("FLASH_SVD_TRUST_PICKLE", raising=False)
    torch.save([1, 2, 3], tmp_path / "x.pt")
    with pytest.raises(ValueError, match="Unrecognized checkpoint format"):
        DS.get_model_from_local(str(tmp_path / "x.pt"))
    # objects are unpickled only from a file the caller trusts
    torch.save(nn.Linear(2, 2), tmp_path / "m.pt")
    with pytest.raises(RuntimeError, match="Refusing to load pickled checkpoint"):
        DS.get_model_from_local(str(tmp_path / "m.pt"))
    monkeypatch.setenv("FLASH_SVD_TRUST_PICKLE", "1")
    with pytest.raises(ValueError, match="could not recover a tokenizer"):
        DS.get_model_from_local(str(tmp_path / "m.pt"))
    monkeypatch.delenv("FLASH_SVD_TRUST_PICKLE")
    torch.save(nn.Linear(2, 2), tmp_path / "llama_svdllm_0.5.pt")        # named like the compression scripts' outputs
    with pytest.raises(ValueError, match="could not recover a tokenizer"):
        DS.get_model_from_local(str(tmp_path / "llama_svdllm_0.5.pt"))


def test_pickle_shims_exist_only_during_a_load():
    import sys

    import transformers.activations as act

    had = hasattr(act, "SiLUActivation")
    with CK.pickle_compat_shims():
        assert hasattr(act, "SiLUActivation")
        layer = sys.modules["modules.module"].SVDTransformLayer(1, two=2)
        assert isinstance(layer, nn.Module)
        assert float(act.SiLUActivation()(torch.tensor(0.0))) == 0.0
    assert hasattr(act, "SiLUActivation") == had
    assert "modules.module" not in sys.modules


# ---- pinned against the reference's own helpers (tests/golden/make_checkpoint_golden.py ran them)
def _golden():
    from pathlib import Path

    return json.loads((Path(__file__).parent / "golden" / "checkpoint_format_cases.json").read_text())


def test_key_sets_and_destinations_match_the_reference_functions():
    g = _golden()
    assert sorted(CK.expected_basis_sharing_keys(2)) == g["expected_keys_2_layers"]
    assert len(g["destination"]) >= 40
    for key, want in g["destination"].items():
        assert CK.basis_sharing_destination(key) == want, key
    for raw, want in g["is_basis_sharing"].items():
        assert CK.is_basis_sharing_config(json.loads(raw)) == want, raw
    for raw, want in g["dtype"].items():
        assert str(CK._DTYPES.get(raw.strip().lower())) == want, raw


def test_shard_discovery_matches_the_reference_function(tmp_path):
    g = _golden()["shards"]

    def names():
        try:
            return [p.name for p in CK.iter_weight_shards(tmp_path)]
        except Exception as e:
            return f"{type(e).__name__}: {str(e).replace(str(tmp_path), '<dir>')}"

    assert names() == g["empty"]
    for n in ("pytorch_model-00003-of-00003.bin", "pytorch_model-00001-of-00003.bin", "pytorch_model-00002-of-00003.bin"):
        (tmp_path / n).write_bytes(b"")
    assert names() == g["numbered"]
    (tmp_path / "pytorch_model.bin").write_bytes(b"")
    assert names() == g["single_wins_over_numbered"]
    index = tmp_path / "pytorch_model.bin.index.json"
    index.write_text(json.dumps({"weight_map": {"b": "pytorch_model-00002-of-00003.bin", "a": "pytorch_model-00003-of-00003.bin",
                                                "c": "pytorch_model-00002-of-00003.bin"}}))
    assert names() == g["index_order_of_first_mention"]
    index.write_text(json.dumps({"weight_map": {"a": "missing.bin"}}))
    assert names() == g["index_missing_file"]
    index.write_text(json.dumps({"weight_map": {}}))
    assert names() == g["index_empty"]


def test_group_tying_and_trust_heuristics_match_the_reference_functions(monkeypatch):
    from transformers import LlamaConfig

    g = _golden()
    cfg = LlamaConfig(**dict(CFG, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                             num_key_value_heads=1, vocab_size=20))
    model = DS.build_svd_llama(cfg)
    L = model.model.layers
    for holder, lin in (("self_attn", "q_v_proj"), ("mlp", "down_v_proj")):
        getattr(getattr(L[1], holder), lin).weight.data.copy_(getattr(getattr(L[0], holder), lin).weight.data)
    CK.tie_basis_groups(model, {"q_groups": [[0, 1]], "down_groups": [[0, 1]], "k_groups": [[0], [1]], "o_groups": "x"})
    got = {"q_v_proj": L[0].self_attn.q_v_proj.weight is L[1].self_attn.q_v_proj.weight,
           "down_v_proj": L[0].mlp.down_v_proj.weight is L[1].mlp.down_v_proj.weight,
           "k_v_proj": L[0].self_attn.k_v_proj.weight is L[1].self_attn.k_v_proj.weight,
           "o_v_proj": L[0].self_attn.o_v_proj.weight is L[1].self_attn.o_v_proj.weight}
    assert got == g["tied"]
    with pytest.raises(ValueError) as e:
        CK.tie_basis_groups(DS.build_svd_llama(cfg), {"up_groups": [[0, 1]]})
    assert str(e.value).split("max diff")[0] == g["tie_errors"]["not_shared"].split("max diff")[0]
    bad = DS.build_svd_llama(cfg)
    bad.model.layers[1].mlp.gate_v_proj = nn.Linear(32, 4, bias=False)
    with pytest.raises(ValueError) as e:
        CK.tie_basis_groups(bad, {"gate_groups": [[0, 1]]})
    assert str(e.value) == g["tie_errors"]["shape"]
    # file names the reference treats as its own outputs (it also asks that the file lies inside its
    # checkout; this package looks at the name only)
    monkeypatch.delenv("FLASH_SVD_TRUST_PICKLE", raising=False)
    for name, want in g["trusted_name"].items():
        assert CK.is_trusted_pickle("/somewhere/" + name) == want, name
