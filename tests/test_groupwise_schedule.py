"""The tile scheduler of the group-scaled FP8 CTA-pair kernel, run on the host (the kernel's own code, compiled for
both sides): every output element of every row group is covered exactly once, whole tiles come before the pieces of
the cut last round, and a piece is the last item of its pair."""
import ctypes

import numpy as np
import pytest

from dsl_tool_b200 import _lib


def _schedule(offs, m_total, n, pairs, band=0, whole=0):
    lib = _lib.lib()
    cap = 1 << 16
    out = np.zeros((cap, 6), np.int32)
    if offs is None:
        po, g = None, 1
    else:
        arr = np.ascontiguousarray(offs, np.int32)
        po, g = arr.ctypes.data_as(ctypes.c_void_p), len(arr) - 1
    cnt = lib.dsl_selftest_groupwise_schedule(po, g, m_total, n, pairs, band, whole, out.ctypes.data_as(ctypes.c_void_p), cap)
    assert cnt >= 0, cnt
    return out[:cnt]


def _check_cover(items, offs, n):
    m_total = int(offs[-1])
    hits = np.zeros((m_total, n), np.uint8)
    for pair, group, row0, row_end, n0, width in items:
        assert row_end == offs[group + 1] and offs[group] <= row0 < row_end and (row0 - offs[group]) % 256 == 0
        assert width in (64, 256) and n0 % width == 0
        r1, c1 = min(row0 + 256, row_end), min(n0 + width, n)
        if n0 < n:
            hits[row0:r1, n0:c1] += 1
    assert (hits == 1).all()


@pytest.mark.parametrize("m,n,pairs", [(4096, 14336, 74), (1024, 14336, 74), (2560, 2000, 74), (8192, 8192, 74),
                                       (300, 256, 74), (19 * 256, 256 * 4, 74), (777, 1000, 3), (5000, 3000, 5)])
def test_dense_cover_and_cut(m, n, pairs):
    items = _schedule(None, m, n, pairs)
    tiles = -(-m // 256) * -(-n // 256)
    rest = tiles % pairs
    cut = tiles > pairs and 0 < rest and 4 * rest <= pairs
    assert len(items) == (tiles - rest + 4 * rest if cut else tiles)
    if m * n <= 1 << 26:
        _check_cover(items, np.array([0, m]), n)
    widths = items[:, 5]
    if cut:
        first = int(np.argmax(widths == 64))
        assert first == tiles - rest and (widths[:first] == 256).all() and (widths[first:] == 64).all()
        piece_pairs = items[first:, 0]
        assert len(set(piece_pairs.tolist())) == len(piece_pairs)              # at most one piece per pair ...
        for p in piece_pairs:                                                  # ... and it is that pair's last item
            assert items[items[:, 0] == p][-1, 5] == 64
    else:
        assert (widths == 256).all()
    whole = _schedule(None, m, n, pairs, whole=1)
    assert len(whole) == tiles and (whole[:, 5] == 256).all()


def test_default_workload_numbers():
    items = _schedule(None, 4096, 14336, 74)
    assert len(items) == 888 + 32 and (items[:888, 5] == 256).all() and (items[888:, 5] == 64).all()


@pytest.mark.parametrize("seed", range(12))
def test_ragged_groups_cover(seed):
    rng = np.random.default_rng(seed)
    g = int(rng.integers(1, 9))
    sizes = rng.integers(0, 900, g)
    sizes[rng.integers(0, g)] = 0 if g > 1 else sizes[0]                       # an empty group when there are several
    offs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    n = int(rng.integers(1, 12)) * 128 + int(rng.integers(0, 2)) * 40
    pairs = int(rng.choice([3, 7, 74]))
    band = int(rng.choice([0, 1, 3, 8]))
    if offs[-1] == 0:
        assert len(_schedule(offs, 0, n, pairs, band)) == 0
        return
    items = _schedule(offs, int(offs[-1]), n, pairs, band)
    _check_cover(items, offs, n)
    assert (items[:, 0] == np.arange(len(items)) % pairs).all()


def test_argument_errors():
    lib = _lib.lib()
    out = np.zeros((4, 6), np.int32)
    po = out.ctypes.data_as(ctypes.c_void_p)
    assert lib.dsl_selftest_groupwise_schedule(None, 1, 4096, 14336, 74, 0, 0, None, 4) == -1
    assert lib.dsl_selftest_groupwise_schedule(None, 1, 4096, 14336, 0, 0, 0, po, 4) == -2
    assert lib.dsl_selftest_groupwise_schedule(None, 1, 4096, 14336, 74, 0, 0, po, 4) == -6                # too many items
    bad = np.array([0, 10, 5], np.int32)
    assert lib.dsl_selftest_groupwise_schedule(bad.ctypes.data_as(ctypes.c_void_p), 0, 5, 256, 74, 0, 0, po, 4) == -2


@pytest.mark.parametrize("offs,m_total", [
    ([0, 300, 5000], 600),            # last entry beyond the rows there are
    ([0, 400, 100, 600], 600),        # decreasing
    ([-50, 200, 10_000_000], 512),    # negative first entry, absurd last one
    ([700, 650, 640], 600),           # everything out of range
    ([0, 2_000_000_000, -2_000_000_000, 300], 300),
])
def test_malformed_offsets_stay_inside_the_operands(offs, m_total):
    """Row-group offsets are device data the kernel cannot refuse; its sanitiser (entries clamped to [0, m_total],
    each raised to its predecessor) must keep every item's rows inside [0, m_total) and never cover a row twice."""
    n = 512
    items = _schedule(np.array(offs, np.int32), m_total, n, 7)
    hits = np.zeros(m_total, np.int32)
    for pair, group, row0, row_end, n0, width in items:
        assert 0 <= row0 < row_end <= m_total
        if n0 == 0:
            hits[row0:min(row0 + 256, row_end)] += 1
    assert hits.max(initial=0) <= 1
    # the sanitised table: clamp, then running maximum
    clean = np.maximum.accumulate(np.clip(np.array(offs, np.int64), 0, m_total))
    assert hits.sum() == clean[-1] - clean[0]
