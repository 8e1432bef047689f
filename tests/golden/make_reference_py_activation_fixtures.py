"""Generates tests/golden/reference_py_activations.npz from the reference's CPU-runnable gated activations
(`TiledSwiGLU`, `TiledGeGLU` in tilelang/activations/activation_kernels.py:38-90), imported read-only from the
reference tree.  Run where the reference is mounted:

    python tests/golden/make_reference_py_activation_fixtures.py [--reference /path/to/reference]

The fixture pins the oracle's `swiglu` / `geglu` (oracle/quant_oracle.py), which in turn check the fused
epilogue of the gate/up GEMM.  Inputs: seeded N(0, 2) values plus the points where the formulas are touchy
(0, +-0, large magnitudes either side).
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def load_reference(root):
    path = os.path.join(root, "tilelang", "activations", "activation_kernels.py")
    spec = importlib.util.spec_from_file_location("_reference_tilelang_activations", path)
    mod = importlib.util.module_from_spec(spec)
    sys.dont_write_bytecode = True
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "reference_py_activations.npz"))
    args = ap.parse_args()
    ref = load_reference(args.reference)
    rng = np.random.default_rng(11)
    B, H = 12, 40
    x = (rng.standard_normal((B, 2 * H)) * 2).astype(np.float32)
    x[0, :8] = [0.0, -0.0, 1e-6, -1e-6, 30.0, -30.0, 88.0, -88.0]          # gate values
    x[0, H:H + 8] = [1.0, 1.0, 1.0, 1.0, 2.0, 2.0, -1.0, -1.0]             # matching up values
    t = torch.from_numpy(x)
    out = dict(x=x, swiglu=ref.TiledSwiGLU().forward(t).numpy(), geglu=ref.TiledGeGLU().forward(t).numpy())
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
