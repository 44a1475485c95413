"""CPU: the C-ABI library loads and exports every symbol declared in include/flashsvd_b200.h.
No compute call is made (there is no GPU here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "flashsvd_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fsvd_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path_entry_points():
    names = declared_symbols()
    for need in ("fsvd_mlp_swiglu_decode", "fsvd_qkv_rope_append", "fsvd_flash_decode",
                 "fsvd_lowrank_proj", "fsvd_decode_layer", "fsvd_model_step"):
        assert need in names


def test_library_exports_every_declared_symbol():
    from flashsvd_b200 import _lib

    if not _lib.LIB_PATH.exists():
        from flashsvd_b200 import build

        build.build()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    assert lib.fsvd_version() >= 100


def test_binding_covers_the_header():
    from flashsvd_b200 import _lib

    assert sorted(_lib.EXPORTS) == declared_symbols()


def test_ops_refuse_cpu_tensors():
    import torch

    from flashsvd_b200 import ops

    with pytest.raises(ValueError):
        ops._ptr(torch.zeros(4))
