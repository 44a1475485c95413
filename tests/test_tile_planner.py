"""CPU: host arithmetic of the tiled path's planner through the library's debug entry points: the K
split of a GEMM (segments = CTAs of a cluster) and the segment count shared by the q / k / v lifts."""
import ctypes as C

import pytest

from flashsvd_b200 import _lib


def _split(tiles, nkb, sms=148):
    lib = _lib.load()
    segs, kbs = C.c_int(0), C.c_int(0)
    lib.fsvd_tile_debug_split_k(tiles, nkb, sms, C.byref(segs), C.byref(kbs))
    return segs.value, kbs.value


def test_k_split_invariants_over_a_grid_of_shapes():
    for tiles in (1, 2, 3, 8, 11, 14, 22, 24, 32, 43, 64, 86, 250, 1024):
        for nkb in (1, 2, 3, 4, 5, 7, 8, 16, 21, 23, 43, 56, 64, 128, 172, 448):
            segs, kbs = _split(tiles, nkb)
            assert 1 <= segs <= 8 and kbs >= 1
            assert segs * kbs >= nkb                      # the segments cover K
            assert (segs - 1) * kbs < nkb                 # and none of them is empty
            if segs > 1:
                assert kbs >= 4 or nkb < 8                # a CTA keeps at least 4 k-blocks (64 KB of factor) where K has them
            assert tiles * segs <= 148 + tiles // 2 + tiles or segs == 1   # about one CTA per SM


def test_measured_shapes_keep_their_split():
    # shapes of the 7B and the 8-way sharded 70B layer, as they were profiled
    assert _split(64, 21)[0] == 2 and _split(64, 43)[0] == 2       # o_lift / down_lift of a 70B shard: 64 x 2
    assert _split(43, 128)[0] == 3 and _split(22, 56)[0] == 7      # mlp_rank 43 x 3, down_rank 22 x 7
    assert _split(14, 128)[0] == 8 and _split(11, 16)[0] == 4      # qkv_rank 14 x 8, o_rank 11 x 4
    assert _split(32, 16)[0] == 4 and _split(86, 24)[0] == 2       # 7B: o_lift 32 x 4, gate + up lifts 86 x 2


@pytest.mark.parametrize("nkb,segs,want", [((21, 4, 4), (5, 1, 1), 4), ((21, 4, 4), (2, 1, 1), 2), ((16, 16, 16), (4, 4, 4), 4),
                                           ((2, 1, 1), (1, 1, 1), 0), ((5, 5, 3), (5, 5, 3), 3), ((7, 5, 5), (4, 3, 3), 3), ((9, 2, 2), (2, 1, 1), 2)])
def test_common_segment_count_of_the_three_lifts(nkb, segs, want):
    lib = _lib.load()
    got = lib.fsvd_tile_debug_common_segments(*nkb, *segs)
    assert got == want
    if got:
        for n in nkb:                                    # every K range is cut into exactly `got` non-empty segments
            kbs = -(-n // got)
            assert -(-n // kbs) == got
