"""ctypes binding of libflashsvd_b200.so (the C ABI declared in include/flashsvd_b200.h).

The library is the only compute path of this package: if it is missing or cannot be loaded the
import of any op fails with an error; there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libflashsvd_b200.so"

DTYPE_BF16 = 0
DTYPE_F32 = 1
DTYPE_BF16_Q4 = 2   # bf16 activations, int4-g128 factor tile streams

EXPORTS = (
    "fsvd_version", "fsvd_last_error_string", "fsvd_device_props", "fsvd_set_launch_config",
    "fsvd_workspace_bytes", "fsvd_workspace_init", "fsvd_workspace_status",
    "fsvd_lowrank_proj", "fsvd_mlp_swiglu_decode", "fsvd_qkv_rope_append", "fsvd_flash_decode",
    "fsvd_decode_layer", "fsvd_model_create", "fsvd_model_destroy", "fsvd_model_step",
    "fsvd_model_buffers", "fsvd_model_status", "fsvd_model_reset_sync", "fsvd_launch_count",
    "fsvd_set_trace_buffer", "fsvd_model_num_stages", "fsvd_lowrank_proj_static", "fsvd_lift",
    "fsvd_q4_packed_bytes", "fsvd_q4_pack", "fsvd_set_wait_limit", "fsvd_workspace_clear_status",
    "fsvd_selftest_wait_timeout", "fsvd_static_status", "fsvd_model_num_barriers",
    "fsvd_exchange_region_bytes", "fsvd_exchange_region_alloc", "fsvd_exchange_region_free",
    "fsvd_exchange_region_export", "fsvd_exchange_region_import", "fsvd_exchange_region_release",
    "fsvd_exchange_create", "fsvd_exchange_destroy", "fsvd_exchange_set_trace", "fsvd_tp_workspace_bytes",
    "fsvd_tp_decode_layer",
)


class FsvdDims(C.Structure):
    _fields_ = [
        ("dtype", C.c_int), ("B", C.c_int), ("d", C.c_int), ("H", C.c_int), ("Hk", C.c_int),
        ("Dh", C.c_int), ("I", C.c_int), ("Rq", C.c_int), ("Rk", C.c_int), ("Rv", C.c_int),
        ("Ro", C.c_int), ("Rg", C.c_int), ("Ru", C.c_int), ("Rd", C.c_int), ("S_max", C.c_int),
        ("vocab", C.c_int), ("n_layers", C.c_int), ("eps", C.c_float),
        ("rows_are_positions", C.c_int),
    ]


LAYER_FIELDS = (
    "ln1_w", "qkv_v", "q_u", "k_u", "v_u", "o_v", "o_u", "ln2_w", "upgate_v", "gate_u", "up_u",
    "down_v", "down_u", "k_cache", "v_cache",
)


class FsvdLayer(C.Structure):
    _fields_ = [(name, C.c_void_p) for name in LAYER_FIELDS]


class FsvdError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"flashsvd_b200 error {code}: {message}")
        self.code = code


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and declare the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("FLASHSVD_B200_LIB", LIB_PATH))
    if not path.exists():
        raise ImportError(
            f"{path} not found: build it with `python -m flashsvd_b200.build` "
            "(nvcc, sm_100a). flashsvd_b200 has no fallback path."
        )
    lib = C.CDLL(str(path))
    vp, ip, sz = C.c_void_p, C.c_int, C.c_size_t
    lib.fsvd_version.restype = ip
    lib.fsvd_last_error_string.restype = C.c_char_p
    lib.fsvd_device_props.argtypes = [C.POINTER(ip), C.POINTER(ip)]
    lib.fsvd_set_launch_config.argtypes = [ip, ip, ip]
    lib.fsvd_workspace_bytes.argtypes = [C.POINTER(FsvdDims)]
    lib.fsvd_workspace_bytes.restype = sz
    lib.fsvd_workspace_init.argtypes = [vp, sz, vp]
    lib.fsvd_workspace_status.argtypes = [vp, C.POINTER(ip)]
    lib.fsvd_lowrank_proj.argtypes = [vp, vp, vp, vp, vp, ip, ip, ip, ip, ip, vp, sz, vp]
    lib.fsvd_lowrank_proj_static.argtypes = [vp, vp, vp, vp, vp, ip, ip, ip, ip, ip, vp]
    lib.fsvd_lift.argtypes = [vp, vp, vp, vp, ip, ip, ip, ip, vp, sz, vp]
    lib.fsvd_mlp_swiglu_decode.argtypes = (
        [vp, vp, C.c_float, vp, vp, vp, vp, vp, vp, vp] + [ip] * 7 + [vp, sz, vp])
    lib.fsvd_qkv_rope_append.argtypes = (
        [vp, vp, C.c_float] + [vp] * 10 + [ip] * 10 + [vp, sz, vp])
    lib.fsvd_flash_decode.argtypes = (
        [vp, vp, vp, vp, ip, vp, ip, ip, ip, ip, ip, C.c_float, ip, vp, sz, vp])
    lib.fsvd_decode_layer.argtypes = [
        C.POINTER(FsvdDims), C.POINTER(FsvdLayer), vp, vp, vp, vp, vp, vp, sz, vp]
    lib.fsvd_model_create.argtypes = [
        C.POINTER(FsvdDims), C.POINTER(FsvdLayer), vp, vp, vp, vp, vp, ip, C.POINTER(vp)]
    lib.fsvd_model_destroy.argtypes = [vp]
    lib.fsvd_model_step.argtypes = [vp, ip, vp]
    lib.fsvd_model_buffers.argtypes = [vp] + [C.POINTER(vp)] * 6
    lib.fsvd_model_status.argtypes = [vp, C.POINTER(ip)]
    lib.fsvd_model_reset_sync.argtypes = [vp, vp]
    lib.fsvd_launch_count.restype = C.c_longlong
    lib.fsvd_set_trace_buffer.argtypes = [vp, sz]
    lib.fsvd_model_num_stages.argtypes = [vp]
    lib.fsvd_q4_packed_bytes.argtypes = [ip, ip]
    lib.fsvd_q4_packed_bytes.restype = sz
    lib.fsvd_q4_pack.argtypes = [vp, vp, vp, ip, ip, vp, vp]
    lib.fsvd_set_wait_limit.argtypes = [C.c_longlong]
    lib.fsvd_workspace_clear_status.argtypes = [vp, vp]
    lib.fsvd_selftest_wait_timeout.argtypes = [vp, sz, vp]
    lib.fsvd_static_status.argtypes = [C.POINTER(ip), ip]
    lib.fsvd_model_num_barriers.argtypes = [vp]
    lib.fsvd_exchange_region_bytes.argtypes = [ip, ip, ip]
    lib.fsvd_exchange_region_bytes.restype = sz
    lib.fsvd_exchange_region_alloc.argtypes = [sz, C.POINTER(vp)]
    lib.fsvd_exchange_region_free.argtypes = [vp]
    lib.fsvd_exchange_region_export.argtypes = [vp, C.c_char_p]
    lib.fsvd_exchange_region_import.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.fsvd_exchange_region_release.argtypes = [vp]
    lib.fsvd_exchange_create.argtypes = [ip, ip, C.POINTER(vp), ip, ip, vp, C.POINTER(vp)]
    lib.fsvd_exchange_destroy.argtypes = [vp]
    lib.fsvd_exchange_set_trace.argtypes = [vp, vp, sz]
    lib.fsvd_tp_workspace_bytes.argtypes = [C.POINTER(FsvdDims)]
    lib.fsvd_tp_workspace_bytes.restype = sz
    lib.fsvd_tp_decode_layer.argtypes = [
        C.POINTER(FsvdDims), C.POINTER(FsvdLayer), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if fn.restype is C.c_int and name not in ("fsvd_version",):
            fn.restype = C.c_int
    _lib = lib
    return lib


def check(status: int) -> None:
    """Map a C status to the reference's error convention (exceptions raised before launch)."""
    if status >= 0:
        return
    msg = load().fsvd_last_error_string().decode("utf-8", "replace")
    if status in (-1, -2, -3, -4):
        raise ValueError(f"flashsvd_b200: {msg}")
    if status == -7:   # the reference's dense cache raises IndexError when it is full
        raise IndexError(f"flashsvd_b200: {msg}")
    raise FsvdError(status, msg)
