"""Generates tests/golden/reference_py.npz from the reference's own CPU-runnable emulation
(`fp8_gemm_tiled`, `grouped_gemm_tiled` in tilelang/gemm/gemm_kernels.py:96-133), imported
read-only from the reference tree.  Run where the reference is mounted:

    python tests/golden/make_reference_py_fixtures.py [--reference /path/to/reference]

Inputs are E4M3 / bf16 code points produced by the oracle's quantisers on seeded data, so the
fixture pins the GEMM step `(A.float() @ B.float()) * scale_a * scale_b` on quantised operands.
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import quant_oracle as O  # noqa: E402


def load_reference(root):
    path = os.path.join(root, "tilelang", "gemm", "gemm_kernels.py")
    spec = importlib.util.spec_from_file_location("_reference_tilelang_gemm", path)
    mod = importlib.util.module_from_spec(spec)
    sys.dont_write_bytecode = True
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "reference_py.npz"))
    args = ap.parse_args()
    ref = load_reference(args.reference)
    rng = np.random.default_rng(7)
    out = {}
    # FP8 per-tensor, ragged sizes (not multiples of the 64x64x32 tiles the reference loops over)
    M, N, K = 150, 200, 176
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    qa, sa = O.quant_fp8_per_tensor(a)
    qb, sb = O.quant_fp8_per_tensor(b)
    A8 = torch.from_numpy(qa).view(torch.float8_e4m3fn)
    B8 = torch.from_numpy(qb).view(torch.float8_e4m3fn)
    c = ref.fp8_gemm_tiled(A8, B8, float(sa), float(sb))
    out.update(fp8_qa=qa, fp8_qb_kn=qb, fp8_sa=np.float32(sa), fp8_sb=np.float32(sb), fp8_c=c.numpy())
    # grouped, fixed-size groups, bf16 operands
    G, M, N, K = 3, 70, 96, 80
    ga = torch.from_numpy(rng.standard_normal((G, M, K)).astype(np.float32)).bfloat16()
    gb = torch.from_numpy(rng.standard_normal((G, K, N)).astype(np.float32)).bfloat16()
    gc = ref.grouped_gemm_tiled(ga, gb)
    out.update(grp_a_bf16_bits=ga.view(torch.int16).numpy(), grp_b_bf16_bits=gb.view(torch.int16).numpy(),
               grp_c=gc.numpy())
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: getattr(v, "shape", None) for k, v in out.items()})


if __name__ == "__main__":
    main()
