"""Shared helpers of the test-suite: seeded inputs, oracle-side references, comparisons."""
import ctypes
import os

import numpy as np

from oracle import quant_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REL_FROB_TOL = 1e-3          # the north-star bound on the fp32 result
BF16_REL_FROB_TOL = 4e-3     # one bf16 rounding is ~1.7e-3 relative Frobenius on its own


def vp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def activations(rng, m, k, outliers=False):
    x = rng.standard_normal((m, k)).astype(np.float32)
    if outliers:   # 0.1 % of the elements at +-20 sigma
        mask = rng.random((m, k)) < 1e-3
        x[mask] = np.where(rng.random(mask.sum()) < 0.5, -20.0, 20.0).astype(np.float32)
    return x


def weights(rng, n, k, std=0.02):
    return (rng.standard_normal((n, k)) * std).astype(np.float32)


def grouped_matmul(A, B_gnk, offsets):
    """A [M,K] x per-group weights [G,N,K] -> [M,N], fp32 accumulate."""
    G, N, _ = B_gnk.shape
    out = np.zeros((A.shape[0], N), dtype=np.float32)
    for g in range(G):
        r0, r1 = int(offsets[g]), int(offsets[g + 1])
        if r1 > r0:
            out[r0:r1] = A[r0:r1] @ B_gnk[g].T
    return out


def moe_offsets(rng, tokens, experts, topk, bias_std=0.0):
    """Routed-row offsets of a softmax/top-k router over seeded N(0,1) logits (+ optional
    per-expert bias to skew the load)."""
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    if bias_std > 0:
        logits += (rng.standard_normal(experts) * bias_std).astype(np.float32)[None, :]
    top = np.argpartition(-logits, topk - 1, axis=1)[:, :topk]
    counts = np.bincount(top.reshape(-1), minlength=experts)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def bf16_ulp_close(got_f32, want_f32, ulps=1):
    """|got - want| <= ulps bf16 ulp of want (both already bf16-representable)."""
    want = np.asarray(want_f32, np.float32)
    got = np.asarray(got_f32, np.float32)
    e = np.frexp(np.maximum(np.abs(want), np.float32(2.0 ** -126)))[1].astype(np.int64)   # |want| in [2^(e-1), 2^e)
    ulp = np.ldexp(1.0, (e - 8).astype(np.int32))
    return np.abs(got.astype(np.float64) - want.astype(np.float64)) <= ulps * ulp


rel_frobenius = O.rel_frobenius
