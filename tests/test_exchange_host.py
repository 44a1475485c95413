"""CPU: host side of the tensor-parallel exchange — region geometry (the Python mirror against the
library) and argument checks that come back before any device call."""
import ctypes as C

import pytest

from flashsvd_b200 import _lib
from flashsvd_b200 import tensor_parallel as TP


@pytest.mark.parametrize("world,rows,d", [(1, 1, 8), (2, 8, 256), (8, 8, 8192), (8, 128, 8192), (4, 3, 4104)])
def test_region_layout_mirrors_the_library(world, rows, d):
    lib = _lib.load()
    lay = TP.region_layout(world, rows, d)
    assert lay["total"] == int(lib.fsvd_exchange_region_bytes(world, rows, d))
    assert lay["flags"] == 256 and lay["slots"] % 256 == 0 and lay["slot_bytes"] >= rows * d * 2
    assert lay["flag_cap"] >= (d + 127) // 128 * 8      # one flag per CTA of the pushing GEMM: row tiles x <= 8 segments
    assert lay["slots"] >= lay["flags"] + 2 * world * lay["flag_cap"] * 4


def test_region_bytes_rejects_bad_geometry():
    lib = _lib.load()
    assert lib.fsvd_exchange_region_bytes(0, 8, 256) == 0
    assert lib.fsvd_exchange_region_bytes(9, 8, 256) == 0      # at most 8 ranks
    assert lib.fsvd_exchange_region_bytes(2, 0, 256) == 0
    with pytest.raises(ValueError):
        TP.PeerExchange(rank=0, world=9, max_rows=8, d=256, regions=[0] * 9)


def test_exchange_create_checks_arguments_before_touching_the_device():
    lib = _lib.load()
    h = C.c_void_p()
    one = (C.c_void_p * 1)(4096)
    two = (C.c_void_p * 2)(4096, 0)
    odd = (C.c_void_p * 1)(4096 + 16)
    assert lib.fsvd_exchange_create(1, 1, one, 8, 256, None, C.byref(h)) == -1      # rank outside the world
    assert lib.fsvd_exchange_create(0, 1, one, 0, 256, None, C.byref(h)) == -1      # no rows
    assert lib.fsvd_exchange_create(0, 1, one, 8, 260, None, C.byref(h)) == -1      # width not a multiple of 8
    assert lib.fsvd_exchange_create(0, 2, two, 8, 256, None, C.byref(h)) == -3      # a region is missing
    assert lib.fsvd_exchange_create(0, 1, odd, 8, 256, None, C.byref(h)) == -3      # not 256-byte aligned
    assert b"aligned" in lib.fsvd_last_error_string()
    assert h.value is None


def test_shard_ranges_and_layer_constructor_errors():
    with pytest.raises(ValueError):
        TP.shard_ranges(8, 2, 64, 640, 0, 3)        # heads do not split over 3 ranks
    sq, sk, si = TP.shard_ranges(64, 8, 128, 28672, 7, 8)
    assert (sq.start, sq.stop) == (7 * 1024, 8 * 1024) and (sk.start, sk.stop) == (7 * 128, 8 * 128)
    assert (si.start, si.stop) == (7 * 3584, 8 * 3584)


def test_tp_layer_entry_rejects_null_arguments_before_any_launch():
    lib = _lib.load()
    dims = _lib.FsvdDims()
    layer = _lib.FsvdLayer()
    assert lib.fsvd_tp_decode_layer(C.byref(dims), C.byref(layer), None, None, None, None, None, None, None, None, None,
                                    None, 0, None) == -1
    assert lib.fsvd_exchange_set_trace(None, None, 0) == -1


def test_trace_summary_arithmetic():
    import torch

    ex = object.__new__(TP.PeerExchange)
    ex._trace = None
    assert ex.trace_summary() == {"exchanges": 0}
    t = torch.zeros(8, 3, dtype=torch.int64)
    base = 1_000_000
    for i, (wait_ns, red_ns) in enumerate(((2000, 5000), (1000, 4000), (3000, 6000), (50000, 5000))):
        t[i] = torch.tensor([base, base + wait_ns, base + wait_ns + red_ns])
    ex._trace = t                                     # four records written, four still empty
    s = ex.trace_summary()
    assert s["exchanges"] == 4 and s["wait_us_max"] == 50.0
    assert s["wait_us_median"] == pytest.approx(2.5) and s["reduce_us_median"] == pytest.approx(5.0)
