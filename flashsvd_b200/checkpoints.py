"""Local checkpoint formats of the reference -> models made of this package's low-rank modules.

Three on-disk / in-memory forms reach the reference's decode path besides the plain factored
state dict (utils/model_utils.py:850-901 dispatches between them):

* **Basis-sharing export** (utils/model_utils.py:271-522): a Hugging Face directory whose
  ``config.json`` names a ``ShareLlama...`` architecture, ``pytorch_model.bin`` (one file, numbered
  shards, or an index with a ``weight_map``) with keys ``...self_attn.q_proj.weight`` (the output-side
  factor, ``q_u_proj`` here) and ``...self_attn.q_basis.weight`` (the input-side factor,
  ``q_v_proj``), likewise k / v / o and ``mlp.gate / up / down``; ``q_groups`` ... ``down_groups`` in
  the config list the layers that share one basis.  The loader checks that every expected tensor
  arrived, that the members of a group really hold equal bases, ties them to ONE parameter (the
  decode engine then keeps one device buffer per group), and requires equal q / k / v ranks and equal
  gate / up ranks, as the reference does.
* **Wrapped factor pairs** (utils/model_utils.py:525-671): a Llama whose ``q_proj`` ... ``down_proj``
  are modules holding two ``nn.Linear``: ``u_proj`` / ``v_proj``, or ``BLinear`` / ``ALinear`` (the
  Dobi-SVD naming, B = output side).  They are replaced by ``SVD_LlamaAttention`` / ``SVD_LlamaMLP``
  that share the same weight storage.
* ``torch.save({'model': model, 'tokenizer': tokenizer})`` and a pickled model object: handled in
  ``demo_support.get_model_from_local``, which passes the model through the conversion above.
  Such files are pickles: ``torch_load_local_checkpoint`` first tries the tensors-only load and
  unpickles objects only from a file the caller trusts (``FLASH_SVD_TRUST_PICKLE=1``, or a file name
  that looks like an output of the reference's own compression scripts), as
  utils/model_utils.py:943-1090 does.

Everything here is host-side Python on CPU tensors; nothing is computed.
"""
from __future__ import annotations

import contextlib
import json
import os
import sys
import types
from pathlib import Path
from typing import Dict, Iterator, Optional

import torch
import torch.nn as nn

ATTN_KEYS = {"q_proj": "q_u_proj", "q_basis": "q_v_proj", "k_proj": "k_u_proj", "k_basis": "k_v_proj",
             "v_proj": "v_u_proj", "v_basis": "v_v_proj", "o_proj": "o_u_proj", "o_basis": "o_v_proj"}
MLP_KEYS = {"gate_proj": "gate_u_proj", "gate_basis": "gate_v_proj", "up_proj": "up_u_proj", "up_basis": "up_v_proj",
            "down_proj": "down_u_proj", "down_basis": "down_v_proj"}
GROUPS = {"q_groups": ("self_attn", "q_v_proj"), "k_groups": ("self_attn", "k_v_proj"), "v_groups": ("self_attn", "v_v_proj"),
          "o_groups": ("self_attn", "o_v_proj"), "gate_groups": ("mlp", "gate_v_proj"), "up_groups": ("mlp", "up_v_proj"),
          "down_groups": ("mlp", "down_v_proj")}
_DTYPES = {"torch.float16": torch.float16, "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
           "torch.bfloat16": torch.bfloat16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "torch.float32": torch.float32, "float32": torch.float32, "fp32": torch.float32}


def read_local_config(path: Path) -> Dict[str, object]:
    """config.json of a directory as a dict ({} when absent or unreadable; utils/model_utils.py:163-172)."""
    try:
        data = json.loads((Path(path) / "config.json").read_text(encoding="utf-8"))
    except Exception:
        return {}
    return data if isinstance(data, dict) else {}


def is_basis_sharing_config(cfg: Dict[str, object]) -> bool:
    """An architecture name containing "sharellama" marks the export (utils/model_utils.py:202-206)."""
    archs = cfg.get("architectures")
    return isinstance(archs, list) and any("sharellama" in str(a).lower() for a in archs)


def iter_weight_shards(path: Path) -> Iterator[Path]:
    """The ``pytorch_model*.bin`` files of a directory in loading order: those of the index's
    ``weight_map`` (each once, in order of first mention), else the single file, else the numbered
    shards sorted by name (utils/model_utils.py:241-268)."""
    path = Path(path)
    index = path / "pytorch_model.bin.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text(encoding="utf-8")).get("weight_map")
        if not isinstance(weight_map, dict) or not weight_map:
            raise ValueError(f"Invalid HF shard index at: {index}")
        for name in dict.fromkeys(str(v) for v in weight_map.values()):
            shard = path / name
            if not shard.is_file():
                raise FileNotFoundError(f"Missing shard referenced by index: {shard}")
            yield shard
        return
    single = path / "pytorch_model.bin"
    if single.is_file():
        yield single
        return
    shards = sorted(path.glob("pytorch_model-*.bin"))
    if not shards:
        raise FileNotFoundError(f"Could not find HF PyTorch checkpoint shards under: {path}")
    yield from shards


def expected_basis_sharing_keys(num_hidden_layers: int) -> set:
    keys = {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"}
    for li in range(int(num_hidden_layers)):
        pre = f"model.layers.{li}"
        keys.update({f"{pre}.input_layernorm.weight", f"{pre}.post_attention_layernorm.weight"})
        keys.update(f"{pre}.self_attn.{k}.weight" for k in ATTN_KEYS)
        keys.update(f"{pre}.mlp.{k}.weight" for k in MLP_KEYS)
    return keys


def basis_sharing_destination(key: str) -> Optional[str]:
    """State-dict key of this package's model for a key of the export (None: not a tensor of the
    model, it is skipped; utils/model_utils.py:302-363)."""
    if key in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"):
        return key
    parts = key.split(".")
    if len(parts) < 5 or parts[0] != "model" or parts[1] != "layers" or not parts[2].isdigit():
        return None
    if parts[3] in ("input_layernorm", "post_attention_layernorm") and parts[4:] == ["weight"]:
        return key
    if len(parts) != 6 or parts[5] != "weight":
        return None
    table = ATTN_KEYS if parts[3] == "self_attn" else MLP_KEYS if parts[3] == "mlp" else {}
    dst = table.get(parts[4])
    return None if dst is None else ".".join(parts[:4] + [dst, "weight"])


def _llama_config(raw: Dict[str, object]):
    from transformers import LlamaConfig

    skip = ("architectures", "model_type", "auto_map", "torch_dtype", "dtype") + tuple(GROUPS)
    return LlamaConfig(**{k: v for k, v in raw.items() if k not in skip})


def load_basis_sharing_dir(path, cfg: Optional[Dict[str, object]] = None):
    """The model of a basis-sharing export directory (tokenizer handling is the caller's)."""
    from .demo_support import build_svd_llama

    path = Path(path)
    cfg = read_local_config(path) if cfg is None else cfg
    config = _llama_config(cfg)
    expected = expected_basis_sharing_keys(int(config.num_hidden_layers))
    state, seen = {}, set()
    for shard_path in iter_weight_shards(path):
        shard = torch.load(str(shard_path), map_location="cpu", weights_only=True)
        if not isinstance(shard, dict):
            raise TypeError(f"Unexpected shard type for {shard_path}: {type(shard)!r}")
        for key, tensor in shard.items():
            dst = basis_sharing_destination(str(key))
            if dst is None:
                continue
            if not isinstance(tensor, torch.Tensor):
                raise TypeError(f"Expected a tensor weight, got: {type(tensor)!r}")
            state[dst] = tensor
            seen.add(str(key))
        del shard
    missing = sorted(expected - seen)
    if missing:
        raise KeyError(f"Basis_Sharing load is missing {len(missing)} required tensors from {path}. "
                       f"First missing keys: {', '.join(missing[:8])}")
    dtype = _DTYPES.get(str(cfg.get("torch_dtype") or cfg.get("dtype") or "").strip().lower())
    model = build_svd_llama(config, state)
    if dtype is not None:
        model = model.to(dtype)
    tie_basis_groups(model, cfg)
    finalize_basis_sharing(model)
    model.seqlen = int(getattr(model.config, "max_position_embeddings", 2048))
    return model


def tie_basis_groups(model: nn.Module, cfg: Dict[str, object]) -> None:
    """The layers of a group keep ONE parameter for their shared input-side factor; a group whose
    members differ is an error (utils/model_utils.py:366-406)."""
    layers = model.model.layers
    for group_name, (holder, lin_name) in GROUPS.items():
        raw_groups = cfg.get(group_name)
        if not isinstance(raw_groups, list):
            continue
        for gi, raw in enumerate(raw_groups):
            if not isinstance(raw, list) or len(raw) <= 1:
                continue
            group = [int(i) for i in raw]
            ref = getattr(getattr(layers[group[0]], holder), lin_name)
            for li in group[1:]:
                cur = getattr(getattr(layers[li], holder), lin_name)
                if tuple(cur.weight.shape) != tuple(ref.weight.shape):
                    raise ValueError(f"Basis_Sharing group {group_name}[{gi}] has mismatched shapes: "
                                     f"{tuple(ref.weight.shape)} vs {tuple(cur.weight.shape)}")
                if not torch.equal(cur.weight, ref.weight):
                    diff = float((cur.weight.detach().float() - ref.weight.detach().float()).abs().max())
                    raise ValueError(f"Basis_Sharing group {group_name}[{gi}] is not actually shared "
                                     f"(layers {group[0]} and {li}, max diff {diff:.6f}).")
                cur.weight = ref.weight


def finalize_basis_sharing(model: nn.Module) -> None:
    """Rank checks and the per-module attributes the reference sets (utils/model_utils.py:409-464)."""
    for li, layer in enumerate(model.model.layers):
        attn, mlp = layer.self_attn, layer.mlp
        rq, rk, rv = (int(getattr(attn, n).weight.shape[0]) for n in ("q_v_proj", "k_v_proj", "v_v_proj"))
        if len({rq, rk, rv}) != 1:
            raise ValueError(f"Basis_Sharing attention layer {li} must have shared q/k/v rank; got {rq}/{rk}/{rv}.")
        rg, ru = int(mlp.gate_v_proj.weight.shape[0]), int(mlp.up_v_proj.weight.shape[0])
        if rg != ru:
            raise ValueError(f"Basis_Sharing MLP layer {li} must have shared gate/up rank; got {rg}/{ru}.")
        hidden, inter = int(mlp.up_v_proj.weight.shape[1]), int(mlp.gate_u_proj.weight.shape[0])
        attn.layer_idx, attn.low_rank = li, rq
        attn.ratio = float(2.0 * rq / max(1, hidden))
        attn.use_lowrank_cache = True
        mlp.ratio = float(rg * (float(hidden) + float(inter)) / max(1.0, float(hidden) * float(inter)))


# ---------------------------------------------------------------------------- wrapped factor pairs
def _pair(mod) -> Optional[tuple]:
    """(output-side nn.Linear, input-side nn.Linear) of a wrapped projection, or None."""
    for u_name, v_name in (("u_proj", "v_proj"), ("BLinear", "ALinear")):
        u, v = getattr(mod, u_name, None), getattr(mod, v_name, None)
        if isinstance(u, nn.Linear) and isinstance(v, nn.Linear):
            return u, v
    return None


def _share(dst: nn.Linear, src: nn.Linear) -> None:
    dst.weight = src.weight                      # the same parameter: no copy of the factor
    dst.in_features, dst.out_features = int(src.weight.shape[1]), int(src.weight.shape[0])
    if src.bias is not None and bool(src.bias.detach().ne(0).any()):
        raise ValueError("a low-rank factor with a non-zero bias cannot be expressed by the decode kernels")


def convert_wrapped_factor_pairs(model: nn.Module) -> nn.Module:
    """Layers whose seven projections are wrapped factor pairs get ``SVD_LlamaAttention`` /
    ``SVD_LlamaMLP`` over the same weights; other layers (already native, or dense) are left alone
    (utils/model_utils.py:586-671)."""
    from .modules import SVD_LlamaAttention, SVD_LlamaMLP

    layers = getattr(getattr(model, "model", None), "layers", None)
    if layers is None:
        return model
    names_a, names_m = ("q", "k", "v", "o"), ("gate", "up", "down")
    for li, layer in enumerate(layers):
        attn, mlp = getattr(layer, "self_attn", None), getattr(layer, "mlp", None)
        if attn is None or mlp is None or (hasattr(attn, "q_u_proj") and hasattr(mlp, "gate_u_proj")):
            continue
        pairs = {n: _pair(getattr(attn, f"{n}_proj", None)) for n in names_a}
        pairs.update({n: _pair(getattr(mlp, f"{n}_proj", None)) for n in names_m})
        if any(p is None for p in pairs.values()):
            continue
        ranks = {n: int(p[1].weight.shape[0]) for n, p in pairs.items()}
        if min(ranks.values()) <= 0:
            raise ValueError(f"FlashSVD native conversion found an invalid low-rank projection in layer {li}.")
        cfg = model.config
        new_attn = SVD_LlamaAttention(cfg, ratio=0.5, layer_idx=int(getattr(attn, "layer_idx", li) or li))
        new_mlp = SVD_LlamaMLP(int(cfg.hidden_size), int(cfg.intermediate_size), str(getattr(cfg, "hidden_act", "silu")), ratio=0.5)
        for n in names_a:
            _share(getattr(new_attn, f"{n}_u_proj"), pairs[n][0])
            _share(getattr(new_attn, f"{n}_v_proj"), pairs[n][1])
        for n in names_m:
            _share(getattr(new_mlp, f"{n}_u_proj"), pairs[n][0])
            _share(getattr(new_mlp, f"{n}_v_proj"), pairs[n][1])
        hidden, inter = float(cfg.hidden_size), float(cfg.intermediate_size)
        new_attn.low_rank = ranks["q"]
        new_attn.ratio = float(2.0 * ranks["q"] / max(1, int(cfg.hidden_size)))
        new_attn.use_lowrank_cache = True
        new_mlp.ratio = float(0.5 * (ranks["gate"] + ranks["up"]) * (hidden + inter) / max(1.0, hidden * inter))
        layer.self_attn, layer.mlp = new_attn, new_mlp
    return model


# ---------------------------------------------------------------------------- pickled checkpoints
_OWN_OUTPUT_NAMES = ("_whitening_only_", "_whitening_then_update_", "_update_only_", "_profiling_", "svdllm", "flashsvd",
                     "merge.pt", "dobi")


def is_trusted_pickle(path) -> bool:
    """True when objects may be unpickled from ``path``: the caller said so in the environment, or the
    file is named like an output of the compression scripts (utils/model_utils.py:943-972, 1075-1079)."""
    if os.environ.get("FLASH_SVD_TRUST_PICKLE", "").strip().lower() in ("1", "true", "yes", "on"):
        return True
    name = Path(path).name.lower()
    return any(key in name for key in _OWN_OUTPUT_NAMES)


@contextlib.contextmanager
def pickle_compat_shims():
    """Names that older pickles refer to and today's libraries no longer have, present for the
    duration of a load and removed afterwards (utils/model_utils.py:975-1040):
    ``transformers...modeling_llama.LlamaSdpaAttention``, ``transformers.activations.SiLUActivation``
    and the ``modules.module.SVDTransformLayer`` placeholder of another compression code base."""
    undo = []
    added = []
    try:
        try:
            import transformers.models.llama.modeling_llama as lm

            if not hasattr(lm, "LlamaSdpaAttention"):
                lm.LlamaSdpaAttention = lm.LlamaAttention
                undo.append((lm, "LlamaSdpaAttention"))
        except Exception:
            pass
        try:
            import transformers.activations as act

            if not hasattr(act, "SiLUActivation"):
                act.SiLUActivation = type("SiLUActivation", (nn.Module,), {"forward": lambda self, x: nn.functional.silu(x)})
                undo.append((act, "SiLUActivation"))
        except Exception:
            pass
        for name in ("modules", "modules.module"):
            if name not in sys.modules:
                sys.modules[name] = types.ModuleType(name)
                added.append(name)
        pkg, mod = sys.modules["modules"], sys.modules["modules.module"]
        if not hasattr(mod, "SVDTransformLayer"):
            mod.SVDTransformLayer = type("SVDTransformLayer", (nn.Module,),
                                         {"__init__": lambda self, *a, **k: nn.Module.__init__(self), "__module__": "modules.module"})
            undo.append((mod, "SVDTransformLayer"))
        if getattr(pkg, "module", None) is not mod and "modules" in added:
            pkg.module = mod
        yield
    finally:
        for owner, attr in reversed(undo):
            with contextlib.suppress(Exception):
                delattr(owner, attr)
        for name in reversed(added):
            sys.modules.pop(name, None)


def torch_load_local_checkpoint(path):
    """``torch.load`` of a local file: tensors-only first; objects only from a trusted file
    (utils/model_utils.py:1043-1090)."""
    path = Path(path)
    try:
        return torch.load(str(path), map_location="cpu", weights_only=True)
    except Exception as e:
        msg = str(e)
        if "Weights only load failed" not in msg and "weights_only" not in msg:
            raise
        if not is_trusted_pickle(path):
            raise RuntimeError(
                f"Refusing to load pickled checkpoint with weights_only=False: {path}\n"
                "PyTorch>=2.6 defaults torch.load(weights_only=True), which can't load "
                "our pickled {'model': model, 'tokenizer': tok} format.\n"
                "If you trust this checkpoint, re-run with: FLASH_SVD_TRUST_PICKLE=1") from e
    with pickle_compat_shims():
        return torch.load(str(path), map_location="cpu", weights_only=False)

