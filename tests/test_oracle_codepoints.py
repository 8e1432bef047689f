"""Code-point level checks of the oracle's encoders (CPU)."""
import hashlib
import json
import os

import ml_dtypes
import numpy as np
import pytest

from oracle import quant_oracle as O
from tests.helpers import GOLDEN


def test_e4m3_roundtrip_all_bytes():
    b = np.arange(256, dtype=np.uint8)
    v = O.e4m3_decode(b)
    finite = ~np.isnan(v)
    assert finite.sum() == 254
    enc = O.e4m3_encode(v[finite])
    assert (enc == b[finite]).all()          # includes +-0 (0x00, 0x80) and subnormals
    assert (O.e4m3_encode(np.array([np.nan], np.float32)) & 0x7F) == 0x7F


def test_e4m3_matches_ml_dtypes_and_saturates():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(200000) * s for s in (1e-3, 1.0, 100.0)]).astype(np.float32)
    x = np.clip(x, -448, 448)
    assert (O.e4m3_encode(x) == x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)).all()
    big = np.array([448.0, 449.0, 464.0, 1e9, np.inf, -1e9, -np.inf], np.float32)
    assert O.e4m3_encode(big).tolist() == [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0xFE]


def test_e4m3_rounding_is_nearest_even():
    # halfway between 1.0 (0x38) and 1.125 (0x39) goes to the even mantissa (0x38);
    # halfway between 1.125 and 1.25 (0x3A) goes up to 0x3A
    assert O.e4m3_encode(np.array([1.0625, 1.1875, 2.0 ** -10, 3 * 2.0 ** -10], np.float32)).tolist() == \
        [0x38, 0x3A, 0x00, 0x02]


def test_e2m1_all_nibbles_roundtrip():
    n = np.arange(16, dtype=np.uint8)
    v = O.e2m1_decode(n)
    enc = O.e2m1_encode_rne(v)
    assert (enc[1:8] == n[1:8]).all() and (enc[9:] == n[9:]).all()
    assert enc[0] == 0 and enc[8] == 0          # the table's entry 8 decodes to +0.0
    assert O.e2m1_encode_rne(np.array([-0.0], np.float32))[0] == 8


def test_e2m1_ties():
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
    assert O.e2m1_encode_rne(ties).tolist() == [0, 2, 2, 4, 4, 6, 6]           # to even mantissa
    assert O.e2m1_encode_ref_lut(ties).tolist() == [0, 1, 2, 3, 4, 5, 6]       # to the lower index
    assert O.e2m1_encode_rne(-ties).tolist() == [8, 10, 10, 12, 12, 14, 14]
    assert O.e2m1_encode_ref_lut(-ties).tolist() == [0, 9, 10, 11, 12, 13, 14]
    assert O.e2m1_encode_rne(np.array([6.1, 100, np.inf, -7], np.float32)).tolist() == [7, 7, 7, 15]


def test_e2m1_matches_ml_dtypes_off_ties():
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100000) * 3).astype(np.float32)
    want = np.clip(x, -6, 6).astype(ml_dtypes.float4_e2m1fn).astype(np.float32)
    assert (O.e2m1_decode(O.e2m1_encode_rne(x)) == want).all()


def test_e8m0_and_pack():
    assert O.e8m0_decode(np.array([127, 0, 254], np.uint8)).tolist() == [1.0, 2.0 ** -127, 2.0 ** 127]
    n = np.arange(16, dtype=np.uint8).reshape(1, 16)
    p = O.pack_nibbles(n)
    assert p.tolist() == [[0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]]
    assert (O.unpack_nibbles(p) == n).all()


def test_zero_and_edge_blocks():
    x = np.zeros((4, 64), np.float32)
    q, s = O.quant_fp8_per_tensor(x)
    assert s == np.float32(1e-12) and not q.any()
    p, sf, gs = O.quant_nvfp4(x)
    assert gs == 1.0 and not sf.any() and not p.any()
    p, sf = O.quant_mxfp4(x)
    assert not sf.any() and not p.any()
    x[0, 0] = -3.0                              # one non-zero block; the others stay zero
    p, sf, gs = O.quant_nvfp4(x)
    assert sf[0, 0] == 0x7E and not sf[0, 1:].any() and p[0, 0] == 0x0F   # -6 in the low nibble
    assert (p[1:] == 0).all()
    p, sf = O.quant_mxfp4(x)
    assert sf[0, 0] == 127 - 1 and p[0, 0] == 0x0F                        # 3 = 6 * 2^-1


def test_oracle_known_answers():
    kat = json.load(open(os.path.join(GOLDEN, "kat_oracle.json")))
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    assert O.E4M3_TABLE.view(np.uint32).tolist() == kat["e4m3_decode_table_hex"]
    ties = np.array(kat["e2m1_ties_in"], np.float32)
    assert O.e2m1_encode_rne(ties).tolist() == kat["e2m1_ties_rne"]
    assert O.e2m1_encode_ref_lut(ties).tolist() == kat["e2m1_ties_ref_lut"]
    seeds = {"act_128x256": (11, 128, 256, 1.0), "wgt_160x384": (12, 160, 384, 0.02), "ragged_37x96": (13, 37, 96, 3.0)}
    for name, (seed, m, k, std) in seeds.items():
        x = (np.random.default_rng(seed).standard_normal((m, k)) * std).astype(np.float32)
        x[1, :] = 0.0
        c = kat["cases"][name]
        q, s = O.quant_fp8_per_tensor(x); assert [sha(q), float(s)] == c["fp8_pt"]
        q, s = O.quant_fp8_groupwise(x); assert [sha(q), sha(s)] == c["fp8_1x128"]
        q, s = O.quant_fp8_block(x); assert [sha(q), sha(s)] == c["fp8_128x128"]
        q, sf, gs = O.quant_nvfp4(x)
        assert [sha(q), sha(sf), float(gs), sha(O.swizzle_sf(sf)), q[0, :8].tolist(), sf[0, :4].tolist()] == c["nvfp4"]
        q, sf, gs = O.quant_nvfp4(x, "per_token")
        assert [sha(q), sha(sf), sha(gs), q[0, :8].tolist(), sf[0, :4].tolist(), float(gs[0]), float(gs[1])] == c["nvfp4_per_token"]
        for m in (0, 1, m - 1):                  # the per-token rule is the tensor rule applied to each row alone
            q1, sf1, g1 = O.quant_nvfp4(x[m:m + 1])
            assert (q1[0] == q[m]).all() and (sf1[0] == sf[m]).all() and g1 == gs[m]
        q, sf = O.quant_mxfp4(x)
        assert [sha(q), sha(sf), sha(O.swizzle_sf(sf)), q[0, :8].tolist(), sf[0, :4].tolist()] == c["mxfp4"]
        q, s = O.quant_fp4_ref32(x); assert [sha(q), sha(s)] == c["ref32_lut"]


@pytest.mark.parametrize("rows,nblk", [(1, 1), (128, 4), (129, 5), (300, 37), (4096, 512)])
def test_sf_tiling_roundtrip(rows, nblk):
    rng = np.random.default_rng(rows * 1000 + nblk)
    sf = rng.integers(1, 255, (rows, nblk)).astype(np.uint8)
    buf = O.swizzle_sf(sf)
    assert buf.size == O.sf_swizzled_size(rows, nblk)
    assert (O.unswizzle_sf(buf, rows, nblk) == sf).all()
    # literal formula: byte (r, c) of tile (rt, kt)
    katoms = (nblk + 3) // 4
    for r, b in [(0, 0), (rows - 1, nblk - 1), (rows // 2, nblk // 2)]:
        off = ((r // 128) * katoms + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4
        assert buf[off] == sf[r, b]
    assert buf.sum() == sf.sum()               # padding is zero


def test_sf_tiling_grouped():
    rng = np.random.default_rng(5)
    sf = rng.integers(1, 255, (300, 8)).astype(np.uint8)
    offs = [0, 5, 5, 140, 300]
    buf = O.swizzle_sf_grouped(sf, offs)
    assert buf.size == (1 + 2 + 2) * 2 * 512   # tiles: 1, 0, 2, 2
    assert (O.unswizzle_sf(buf[: 2 * 512], 5, 8) == sf[:5]).all()
    assert (O.unswizzle_sf(buf[2 * 512: 6 * 512], 135, 8) == sf[5:140]).all()
