"""Generates tests/golden/checkpoint_format_cases.json by running the reference's own checkpoint
helpers (utils/model_utils.py) on small inputs.  Needs a FlashSVD checkout; run once in the build
container:

    python tests/golden/make_checkpoint_golden.py --reference <FlashSVD checkout>

Functions of the reference that are executed (nothing of them is copied into this repository):
  _expected_basis_sharing_keys, _assign_basis_sharing_tensor, _tie_basis_sharing_layer_groups,
  _iter_pytorch_bin_shards, _is_basis_sharing_config, _torch_dtype_from_raw,
  _looks_like_flashsvd_checkpoint, _looks_like_dobi_checkpoint.
The model they are applied to is one built from this package's modules (the reference's
models/llama.py is absent from its checkout), so the recorded mapping is "which module weight of
that model the reference fills from which key of an export".
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent / "checkpoint_format_cases.json"

CFG = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
           head_dim=16, vocab_size=20, max_position_embeddings=64, rms_norm_eps=1e-5, hidden_act="silu")


def tiny_model():
    from transformers import LlamaConfig

    from flashsvd_b200.demo_support import build_svd_llama

    return build_svd_llama(LlamaConfig(**CFG))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FLASHSVD_REFERENCE", ""))
    args = ap.parse_args()
    ref = Path(args.reference).resolve()
    sys.path.insert(0, str(ref))
    import utils.model_utils as MU   # the reference's module

    cases = {}
    cases["expected_keys_2_layers"] = sorted(MU._expected_basis_sharing_keys(2))

    # ---- key -> destination: give every key of an export its own constant, let the reference assign it,
    # then look up which parameter of the model holds that constant
    model = tiny_model()
    keys = cases["expected_keys_2_layers"] + ["model.layers.0.self_attn.rotary_emb.inv_freq", "model.layers.1.mlp.act_fn.weight",
                                             "model.layers.0.self_attn.q_proj.bias", "transformer.h.0.attn.weight", "lm_head.bias"]
    accepted = {}
    for i, key in enumerate(keys):
        ok = MU._assign_basis_sharing_tensor(model, key, torch.full((2, 2), float(i + 1)))
        accepted[key] = bool(ok)
    where = {}
    for name, p in model.named_parameters(remove_duplicate=False):
        if tuple(p.shape) == (2, 2):
            where[float(p.flatten()[0])] = name
    cases["destination"] = {key: (where.get(float(i + 1)) if accepted[key] else None) for i, key in enumerate(keys)}

    # ---- group tying: which layers end up with the very same parameter, and the two error texts
    model = tiny_model()
    for l0, l1 in ((0, 1),):
        for holder, lin in (("self_attn", "q_v_proj"), ("mlp", "down_v_proj")):
            a, b = getattr(getattr(model.model.layers[l0], holder), lin), getattr(getattr(model.model.layers[l1], holder), lin)
            b.weight.data.copy_(a.weight.data)
    MU._tie_basis_sharing_layer_groups(model, {"q_groups": [[0, 1]], "down_groups": [[0, 1]], "k_groups": [[0], [1]], "o_groups": "x"})
    L = model.model.layers
    cases["tied"] = {"q_v_proj": L[0].self_attn.q_v_proj.weight is L[1].self_attn.q_v_proj.weight,
                     "down_v_proj": L[0].mlp.down_v_proj.weight is L[1].mlp.down_v_proj.weight,
                     "k_v_proj": L[0].self_attn.k_v_proj.weight is L[1].self_attn.k_v_proj.weight,
                     "o_v_proj": L[0].self_attn.o_v_proj.weight is L[1].self_attn.o_v_proj.weight}
    errors = {}
    try:
        MU._tie_basis_sharing_layer_groups(tiny_model(), {"up_groups": [[0, 1]]})
    except ValueError as e:
        errors["not_shared"] = str(e)
    bad = tiny_model()
    bad.model.layers[1].mlp.gate_v_proj = torch.nn.Linear(32, 4, bias=False)
    try:
        MU._tie_basis_sharing_layer_groups(bad, {"gate_groups": [[0, 1]]})
    except ValueError as e:
        errors["shape"] = str(e)
    cases["tie_errors"] = errors

    # ---- shard discovery
    shard_cases = {}
    with tempfile.TemporaryDirectory() as tmp:
        d = Path(tmp)

        def names():
            try:
                return [p.name for p in MU._iter_pytorch_bin_shards(d)]
            except Exception as e:
                return f"{type(e).__name__}: {str(e).replace(str(d), '<dir>')}"

        shard_cases["empty"] = names()
        for n in ("pytorch_model-00003-of-00003.bin", "pytorch_model-00001-of-00003.bin", "pytorch_model-00002-of-00003.bin"):
            (d / n).write_bytes(b"")
        shard_cases["numbered"] = names()
        (d / "pytorch_model.bin").write_bytes(b"")
        shard_cases["single_wins_over_numbered"] = names()
        (d / "pytorch_model.bin.index.json").write_text(json.dumps({"weight_map": {
            "b": "pytorch_model-00002-of-00003.bin", "a": "pytorch_model-00003-of-00003.bin", "c": "pytorch_model-00002-of-00003.bin"}}))
        shard_cases["index_order_of_first_mention"] = names()
        (d / "pytorch_model.bin.index.json").write_text(json.dumps({"weight_map": {"a": "missing.bin"}}))
        shard_cases["index_missing_file"] = names()
        (d / "pytorch_model.bin.index.json").write_text(json.dumps({"weight_map": {}}))
        shard_cases["index_empty"] = names()
    cases["shards"] = shard_cases

    cases["is_basis_sharing"] = {json.dumps(c): bool(MU._is_basis_sharing_config(c)) for c in (
        {"architectures": ["ShareLlamaForCausalLM"]}, {"architectures": ["LlamaForCausalLM"]}, {"architectures": "ShareLlama"},
        {}, {"architectures": ["x", "my_SHARELLAMA_v2"]})}
    cases["dtype"] = {s: str(MU._torch_dtype_from_raw(s)) for s in ("float16", "torch.bfloat16", "BF16", " fp32 ", "half", "int8", "")}
    names = ("llama_7b_whitening_only_0.8.pt", "x_update_only_.pt", "svdllm_model.pt", "my_FlashSVD.pt", "merge.pt", "model.pt",
             "dobi_llama.pt", "DobiSVD-0.6.pt", "checkpoint.pth", "a_profiling_b.pt", "llama_whitening_then_update_0.5.pt")
    cases["trusted_name"] = {n: bool(MU._looks_like_flashsvd_checkpoint(ref / n) or MU._looks_like_dobi_checkpoint(ref / n)) for n in names}

    OUT.write_text(json.dumps(cases, indent=1, sort_keys=True) + "\n")
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
