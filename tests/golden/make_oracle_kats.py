"""Writes tests/golden/kat_oracle.json: known-answer vectors of the oracle's OWN rules for the
formats the reference does not have (NVFP4, MXFP4, FP8 1x128 / 128x128, scale tiling), so any
later change to those rules is caught.  Code-point tables are stored literally; seeded cases
as SHA-256 of the produced bytes plus a few literal rows.

    python tests/golden/make_oracle_kats.py
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import quant_oracle as O  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def seeded(seed, m, k, std=1.0):
    return (np.random.default_rng(seed).standard_normal((m, k)) * std).astype(np.float32)


def main():
    kat = {}
    kat["e4m3_decode_table_hex"] = O.E4M3_TABLE.view(np.uint32).tolist()
    ties = [0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 0.2499999, 0.2500001, -0.25, -0.75, -0.0, -5.0, -6.5]
    kat["e2m1_ties_in"] = ties
    kat["e2m1_ties_rne"] = O.e2m1_encode_rne(np.array(ties, np.float32)).tolist()
    kat["e2m1_ties_ref_lut"] = O.e2m1_encode_ref_lut(np.array(ties, np.float32)).tolist()
    cases = {}
    for name, (seed, m, k, std) in {"act_128x256": (11, 128, 256, 1.0), "wgt_160x384": (12, 160, 384, 0.02),
                                    "ragged_37x96": (13, 37, 96, 3.0)}.items():
        x = seeded(seed, m, k, std)
        x[1, :] = 0.0
        c = {}
        q, s = O.quant_fp8_per_tensor(x); c["fp8_pt"] = [sha(q), float(s)]
        q, s = O.quant_fp8_groupwise(x); c["fp8_1x128"] = [sha(q), sha(s)]
        q, s = O.quant_fp8_block(x); c["fp8_128x128"] = [sha(q), sha(s)]
        q, sf, gs = O.quant_nvfp4(x); c["nvfp4"] = [sha(q), sha(sf), float(gs), sha(O.swizzle_sf(sf)), q[0, :8].tolist(), sf[0, :4].tolist()]
        q, sf, gs = O.quant_nvfp4(x, "per_token"); c["nvfp4_per_token"] = [sha(q), sha(sf), sha(gs), q[0, :8].tolist(), sf[0, :4].tolist(), float(gs[0]), float(gs[1])]
        q, sf = O.quant_mxfp4(x); c["mxfp4"] = [sha(q), sha(sf), sha(O.swizzle_sf(sf)), q[0, :8].tolist(), sf[0, :4].tolist()]
        q, s = O.quant_fp4_ref32(x); c["ref32_lut"] = [sha(q), sha(s)]
        cases[name] = c
    kat["cases"] = cases
    path = os.path.join(ROOT, "tests", "golden", "kat_oracle.json")
    with open(path, "w") as f:
        json.dump(kat, f, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
