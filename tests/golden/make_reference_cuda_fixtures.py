"""Generates tests/golden/reference_cuda_{ieee,fast}.npz: raw outputs of the reference's own
CUDA kernels (cuda/gemm/fp8_gemm.cu, fp4_gemm.cu, grouped_gemm.cu) on small seeded inputs.

Needs a GPU and the driver binaries built by `make -C oracle ref` (oracle/_ref/ref_*), which
compile the reference's source files unmodified.  Usage:

    python tests/golden/make_reference_cuda_fixtures.py --out <dir>

`ieee` = built without fast-math; `fast` = with the reference's own --use_fast_math flag.
"""
import argparse
import os
import subprocess
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.path.join(ROOT, "oracle", "_ref")

FP8 = dict(M=48, N=40, K=96, G=32)
FP4 = dict(M=32, N=48, K=64)
GRP = dict(G=3, M=40, N=24, K=32, rows=[40, 0, 17])


def make_inputs():
    rng = np.random.default_rng(20240607)
    d = {}
    d["fp8_A"] = (rng.standard_normal((FP8["M"], FP8["K"])) * 1.7).astype(np.float32)
    d["fp8_B"] = (rng.standard_normal((FP8["K"], FP8["N"])) * 0.02).astype(np.float32)
    ng = FP8["K"] // FP8["G"]
    d["fp8_sa"] = rng.uniform(0.5, 2.0, (FP8["M"], ng)).astype(np.float32)
    d["fp8_sb"] = rng.uniform(0.001, 0.01, (ng, FP8["N"])).astype(np.float32)
    d["fp4_A"] = rng.standard_normal((FP4["M"], FP4["K"])).astype(np.float32)
    d["fp4_B"] = (rng.standard_normal((FP4["K"], FP4["N"])) * 0.02).astype(np.float32)
    # exact tie points of the e2m1 grid after scaling: a block whose amax is 6 keeps scale 1
    d["fp4_A"][0, :32] = np.array([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5,
                                   -3.5, -5.0, 0.0, -0.0, 0.5, 1, 1.5, 2, 3, 4, -6, 0.1, 0.3, 0.7, 1.3, 2.2, 2.8,
                                   4.9, 5.1], dtype=np.float32)
    d["fp4_A"][1, :32] = 0.0
    d["grp_A"] = rng.standard_normal((GRP["G"], GRP["M"], GRP["K"])).astype(np.float32)
    d["grp_B"] = rng.standard_normal((GRP["G"], GRP["K"], GRP["N"])).astype(np.float32)
    return d


def run(binary, inputs, args, out_bytes):
    with tempfile.TemporaryDirectory() as tmp:
        fin, fout = os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
        with open(fin, "wb") as f:
            for a in inputs:
                f.write(np.ascontiguousarray(a).tobytes())
        subprocess.run([os.path.join(REF, binary), fin, fout, *map(str, args)], check=True)
        raw = open(fout, "rb").read()
    assert len(raw) == out_bytes, (binary, len(raw), out_bytes)
    return raw


def take(raw, pos, dtype, shape):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    return np.frombuffer(raw[pos:pos + n], dtype=dtype).reshape(shape).copy(), pos + n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden"))
    out_dir = ap.parse_args().out
    os.makedirs(out_dir, exist_ok=True)
    d = make_inputs()
    for variant in ("ieee", "fast"):
        r = dict(d)
        M, N, K, G = FP8["M"], FP8["N"], FP8["K"], FP8["G"]
        raw = run(f"ref_fp8_{variant}", [d["fp8_A"], d["fp8_B"], d["fp8_sa"], d["fp8_sb"]], [M, N, K, G],
                  M * K + K * N + 8 + 2 * M * N * 4)
        p = 0
        r["fp8_qA"], p = take(raw, p, np.uint8, (M, K))
        r["fp8_qB"], p = take(raw, p, np.uint8, (K, N))
        r["fp8_scales"], p = take(raw, p, np.float32, (2,))
        r["fp8_C_per_tensor"], p = take(raw, p, np.float32, (M, N))
        r["fp8_C_groupwise"], p = take(raw, p, np.float32, (M, N))
        M, N, K = FP4["M"], FP4["N"], FP4["K"]
        raw = run(f"ref_fp4_{variant}", [d["fp4_A"], d["fp4_B"]], [M, N, K],
                  M * K // 2 + M * K // 32 * 4 + K * N // 2 + K * N // 32 * 4 + 2 * M * N * 4)
        p = 0
        r["fp4_pA"], p = take(raw, p, np.uint8, (M * K // 2,))
        r["fp4_sA"], p = take(raw, p, np.float32, (M * K // 32,))
        r["fp4_pB"], p = take(raw, p, np.uint8, (K * N // 2,))
        r["fp4_sB"], p = take(raw, p, np.float32, (K * N // 32,))
        r["fp4_C_nvfp4"], p = take(raw, p, np.float32, (M, N))
        r["fp4_C_mxfp4"], p = take(raw, p, np.float32, (M, N))
        G, M, N, K, rows = GRP["G"], GRP["M"], GRP["N"], GRP["K"], GRP["rows"]
        raw = run(f"ref_grouped_{variant}", [d["grp_A"], d["grp_B"]], [G, M, N, K, *rows],
                  (G * M * N + sum(rows) * N) * 4)
        p = 0
        r["grp_C_fixed"], p = take(raw, p, np.float32, (G, M, N))
        r["grp_C_variable"], p = take(raw, p, np.float32, (sum(rows), N))
        r["grp_rows"] = np.array(rows, dtype=np.int32)
        np.savez_compressed(os.path.join(out_dir, f"reference_cuda_{variant}.npz"), **r)
        print("wrote", variant)


if __name__ == "__main__":
    main()
