"""The reference's public helper surface (scripts/demo_support/__init__.py:1-24) on top of this
package: the same names, arguments and result dictionaries, so code written against
``scripts.demo_support`` runs with ``from flashsvd_b200 import demo_support``.

Loading covers the formats that need no network (``get_model_from_local``, utils/model_utils.py:850-901):
a ``torch.save({'model': ..., 'tokenizer': ...})`` file (wrapped factor pairs are converted), a
directory with ``config.json`` + a state dict whose keys carry the ``*_v_proj`` / ``*_u_proj`` factor
names (utils/model_utils.py:637-643), and a basis-sharing export directory (``checkpoints.py``).  Models with
low-rank modules decode through the CUDA library (``generate_text`` builds and keeps a
``DecodeEngine`` for them); any other transformers model takes the plain token loop.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Optional

import torch

from .runtime import configure_runtime, generate_text, runtime_env_snapshot  # noqa: F401

__version__ = "1.5.0"

_DTYPES = {"fp16": torch.float16, "float16": torch.float16, "half": torch.float16, "bf16": torch.bfloat16,
           "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32, "float": torch.float32}


def cast_model_for_inference(model: Any, *, dtype: str = "auto", device=None):
    """dtype "auto": bf16 on CUDA, fp32 on CPU (scripts/demo_support/api.py:146-177)."""
    raw = str(dtype).strip().lower()
    if device is None:
        try:
            target = next(model.parameters()).device
        except StopIteration:
            target = torch.device("cpu")
    else:
        target = torch.device(device)
    if raw == "auto":
        want = torch.bfloat16 if target.type == "cuda" else torch.float32
    elif raw in _DTYPES:
        want = _DTYPES[raw]
    else:
        raise ValueError(f"Unsupported dtype {dtype!r}")
    model = model.to(device=target, dtype=want)
    model.eval()
    return model


def build_svd_llama(config, state_dict: Optional[dict] = None):
    """A transformers LlamaForCausalLM whose layers hold ``SVD_LlamaAttention`` / ``SVD_LlamaMLP``
    with the ranks found in ``state_dict`` (or the rank formula at ``config.flash_svd_ratio``)."""
    from transformers import LlamaForCausalLM

    from .modules import SVD_LlamaAttention, SVD_LlamaMLP

    ratio = float(getattr(config, "flash_svd_ratio", 0.5))
    model = LlamaForCausalLM(config)
    for li, layer in enumerate(model.model.layers):
        attn = SVD_LlamaAttention(config, ratio=ratio, layer_idx=li)
        mlp = SVD_LlamaMLP(config.hidden_size, config.intermediate_size, getattr(config, "hidden_act", "silu"), ratio=ratio)
        if state_dict is not None:
            for mod, holder in ((attn, "self_attn"), (mlp, "mlp")):
                for name, lin in list(mod.named_children()):
                    w = state_dict.get(f"model.layers.{li}.{holder}.{name}.weight")
                    if w is not None and isinstance(lin, torch.nn.Linear) and tuple(w.shape) != tuple(lin.weight.shape):
                        setattr(mod, name, torch.nn.Linear(w.shape[1], w.shape[0], bias=False))
            attn.low_rank = attn.q_u_proj.in_features
        layer.self_attn, layer.mlp = attn, mlp
    if state_dict is not None:
        missing, unexpected = model.load_state_dict(state_dict, strict=False)
        bad = [k for k in missing if "rotary" not in k]
        if bad:
            raise ValueError(f"state dict lacks {len(bad)} tensors, e.g. {bad[:3]}")
    return model


def _local_tokenizer(p: Path):
    if any((p / n).exists() for n in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        try:
            from transformers import AutoTokenizer

            return AutoTokenizer.from_pretrained(str(p), local_files_only=True)
        except Exception:
            return None
    return None


def get_model_from_local(path: str):
    """(model, tokenizer) from a local checkpoint, dispatching as utils/model_utils.py:850-901 does:
    a directory with a basis-sharing export (``checkpoints.load_basis_sharing_dir``); a directory
    with ``config.json`` and ``pytorch_model.bin`` (one file, shards or an index) / ``model.pt``
    holding a factored Llama state dict; a ``torch.save({'model', 'tokenizer'})`` file or a pickled
    model, whose wrapped factor pairs (``u_proj`` / ``v_proj``, ``BLinear`` / ``ALinear``) become
    this package's modules over the same weights."""
    from . import checkpoints

    p = Path(path).expanduser()
    if p.is_dir():
        cfg_path = p / "config.json"
        if not cfg_path.exists():
            raise FileNotFoundError(f"{p} has no config.json")
        raw = checkpoints.read_local_config(p)
        if checkpoints.is_basis_sharing_config(raw):
            return checkpoints.load_basis_sharing_dir(p, raw), _local_tokenizer(p)
        from transformers import LlamaConfig

        config = LlamaConfig(**{k: v for k, v in raw.items() if k not in ("architectures", "model_type", "auto_map")})
        single = next((p / n for n in ("model.pt", "model.bin") if (p / n).exists()), None)
        try:
            files = list(checkpoints.iter_weight_shards(p))
        except FileNotFoundError:
            files = [single] if single is not None else []
        if not files:
            raise FileNotFoundError(f"{p} has no pytorch_model.bin / model.pt")
        sd = {}
        for f in files:
            sd.update(torch.load(f, map_location="cpu", weights_only=True))
        if not any(k.endswith("q_u_proj.weight") for k in sd):
            raise ValueError("the state dict has no *_u_proj / *_v_proj factors: not a FlashSVD Llama export")
        return build_svd_llama(config, sd), _local_tokenizer(p)
    if not p.exists():
        raise FileNotFoundError(str(p))
    obj = checkpoints.torch_load_local_checkpoint(p)
    if isinstance(obj, dict) and "model" in obj:
        return checkpoints.convert_wrapped_factor_pairs(obj["model"]), obj.get("tokenizer")
    if hasattr(obj, "forward"):
        raise ValueError(f"Loaded a model object from {path} but could not recover a tokenizer. "
                         "Please re-save as {'model': model, 'tokenizer': tok}.")
    raise ValueError(f"Unrecognized checkpoint format at: {path}")


def get_model_from_huggingface(name: str, *, hf_token: Optional[str] = None, torch_dtype=None):
    raise RuntimeError(f"{name!r} is not a local path: downloading checkpoints is outside this package "
                       "(pass a local file or directory)")


def get_model_from_source(source: str, *, hf_token: Optional[str] = None, torch_dtype=None):
    raw = str(source).strip()
    local = Path(raw).expanduser()
    if local.exists():
        return get_model_from_local(str(local))
    return get_model_from_huggingface(raw, hf_token=hf_token, torch_dtype=torch_dtype)


def load_for_inference(source: str, *, hf_token: Optional[str] = None, dtype: str = "auto", device="cpu"):
    model, tokenizer = get_model_from_source(source, hf_token=hf_token)
    return cast_model_for_inference(model, dtype=dtype, device=device), tokenizer


@torch.inference_mode()
def decode_kvcache_eval(model, *, prompt_len: int = 2048, new_tokens: int = 128, batch_size: int = 1,
                        device: str = "cuda", warmup: int = 5, max_cache_len: Optional[int] = None, **flags) -> dict:
    """Decode benchmark with the reference's protocol (utils/evaluator.py:272-540): a prompt of
    ``prompt_len`` random tokens fills the cache, ``warmup`` untimed steps, then ``new_tokens`` timed
    single-token steps between CUDA events.  ``model`` is a ``DecodeEngine`` or a model with low-rank
    modules.  Returns the reference's result dictionary (sizes, prefill / decode seconds and tokens/s,
    decode_ms_per_token, the three cache flags)."""
    from .engine import DecodeEngine, engine_for_model

    if flags.get("lowrank_cache", False):
        raise NotImplementedError("lowrank_cache=True selects the reference's rank-space cache mode; flashsvd_b200 serves the "
                                  "dense-cache decode (flashsvd_dense_cache)")
    echo = {k: bool(flags.get(k, False)) for k in ("lowrank_cache", "flashsvd_dense_cache", "baseline_dense_kvcache")}
    if max_cache_len is None:
        max_cache_len = int(prompt_len) + int(warmup) + int(new_tokens) + 1
    eng = model if isinstance(model, DecodeEngine) else engine_for_model(
        model, batch_size=int(batch_size), max_cache_len=int(max_cache_len),
        max_steps=int(prompt_len) + int(warmup) + int(new_tokens) + 8)
    vocab = eng.vocab
    prompt = torch.randint(0, vocab, (eng.B, int(prompt_len)), device=eng.device, dtype=torch.int32)
    eng.reset()
    e0, e1, e2, e3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    e0.record()
    eng.prefill(prompt)
    e1.record()
    if warmup > 0:
        eng.step(int(warmup))
    torch.cuda.synchronize()
    e2.record()
    eng.step(int(new_tokens))
    e3.record()
    torch.cuda.synchronize()
    t_prefill, t_decode = e0.elapsed_time(e1) * 1e-3, e2.elapsed_time(e3) * 1e-3
    if eng.status() != 0:
        raise RuntimeError("a device-side wait ran out during the benchmark")
    inf = float("inf")
    decode_tok_s = eng.B * int(new_tokens) / t_decode if t_decode > 0 else inf
    # the keys of the reference's result (utils/evaluator.py:529-541); decode_tokens_per_s = decode_tok_s
    return {"prompt_len": int(prompt_len), "new_tokens": int(new_tokens), "batch_size": int(eng.B),
            "prefill_time_s": float(t_prefill), "decode_time_s": float(t_decode),
            "prefill_tok_s": eng.B * int(prompt_len) / t_prefill if t_prefill > 0 else inf,
            "decode_tok_s": float(decode_tok_s), "decode_ms_per_token": t_decode * 1000.0 / max(1, int(new_tokens)),
            **echo,   # the flags as passed, like the reference; the cache is the dense [B, S, Hk, Dh] one whatever they say
            "decode_tokens_per_s": float(decode_tok_s)}


__all__ = ["__version__", "cast_model_for_inference", "configure_runtime", "decode_kvcache_eval", "generate_text",
           "get_model_from_huggingface", "get_model_from_local", "get_model_from_source", "load_for_inference",
           "runtime_env_snapshot", "build_svd_llama"]
