"""The oracle's gated activations against outputs of the reference's own CPU implementation
(tests/golden/reference_py_activations.npz, made by make_reference_py_activation_fixtures.py), and
self-consistency of the mixture-of-experts restatement (which has nothing in the reference to pin to)."""
import os

import numpy as np

from oracle import moe_oracle as MO
from oracle import quant_oracle as O
from tests.helpers import GOLDEN


def test_swiglu_and_geglu_match_the_reference_outputs():
    d = np.load(os.path.join(GOLDEN, "reference_py_activations.npz"))
    for name, fn in (("swiglu", O.swiglu), ("geglu", O.geglu)):
        got, want = fn(d["x"]), d[name]
        assert got.shape == want.shape and got.dtype == np.float32
        # one or two ulp where the value is of order 1; where fp32 tanh has saturated (gate < -5) the reference
        # returns exactly 0 and the fp64-evaluated formula 1e-8, hence the absolute term
        assert np.allclose(got, want, rtol=2e-6, atol=2e-6), name
    # the touchy points of row 0: zero gate, tiny gate, saturated sigmoid either side
    assert O.swiglu(d["x"])[0, 0] == 0 and O.swiglu(d["x"])[0, 4] == 60.0 and abs(O.swiglu(d["x"])[0, 5]) < 1e-10


def test_interleaved_form_is_the_same_function():
    rng = np.random.default_rng(2)
    w = rng.standard_normal((3, 10, 7)).astype(np.float32)                   # [G, 2H, K]
    wi = O.interleave_gate_up(w)
    assert np.array_equal(wi[:, 0::2], w[:, :5]) and np.array_equal(wi[:, 1::2], w[:, 5:])
    x = rng.standard_normal((4, 7)).astype(np.float32)
    full, full_i = x @ w[0].T, x @ wi[0].T
    for kind, fn in (("swiglu", O.swiglu), ("geglu", O.geglu)):
        assert np.array_equal(O.gated_of_interleaved(full_i, kind), fn(full))


def test_moe_restatement_is_self_consistent():
    rng = np.random.default_rng(3)
    T, E, k, D = 50, 7, 3, 5
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[0, :3] = 1.5                                                       # a three-way tie: lower indices win, in order
    ids, w = MO.route(logits, k)
    assert list(ids[0]) == [0, 1, 2] if logits[0, 3:].max() < 1.5 else True
    assert np.allclose(w.sum(1), 1, atol=1e-6) and (np.diff(w, axis=1) <= 1e-7).all()
    assert all(len(set(r)) == k for r in ids)
    offsets, tile0, dest = MO.plan(ids, E)
    assert sorted(dest) == list(range(T * k)) and offsets[-1] == T * k
    flat = ids.reshape(-1)
    for e in range(E):                                                        # rows of an expert: its entries, in entry order
        rows = dest[flat == e]
        assert list(rows) == list(range(offsets[e], offsets[e + 1]))
    assert tile0[-1] == sum((offsets[e + 1] - offsets[e] + 127) // 128 for e in range(E))
    tok = MO.token_of_row(dest, k)
    x = rng.standard_normal((T, D))
    y = x[tok]                                                                # identity experts: combine returns sum(w) * x = x
    assert np.allclose(MO.combine(y, ids, w, dest, offsets, 0, E), x, atol=1e-6)
    part = MO.combine(y[offsets[2]:offsets[5]], ids, w, dest, offsets, 2, 5) + MO.combine(y[:offsets[2]], ids, w, dest, offsets, 0, 2) \
        + MO.combine(y[offsets[5]:], ids, w, dest, offsets, 5, E)
    assert np.allclose(part, x, atol=1e-6)                                    # expert ranges partition the sum
