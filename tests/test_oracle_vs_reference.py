"""The oracle against the reference: outputs of the reference's own CUDA kernels captured on a
B200 (tests/golden/reference_cuda_*.npz), of its CPU emulation (tests/golden/reference_py.npz),
and the C restatement of its kernels (oracle/ref_restatement.c).  CPU only."""
import ctypes
import os

import numpy as np
import pytest

from oracle import quant_oracle as O
from tests.helpers import GOLDEN, rel_frobenius, vp


@pytest.fixture(scope="module", params=["ieee", "fast"])
def ref(request):
    return request.param, np.load(os.path.join(GOLDEN, f"reference_cuda_{request.param}.npz"))


def test_fp8_quantiser_bit_exact(ref):
    _, d = ref
    for name, scale in (("A", 0), ("B", 1)):
        q, s = O.quant_fp8_per_tensor(d[f"fp8_{name}"])
        assert (q == d[f"fp8_q{name}"]).all()
        assert s == d["fp8_scales"][scale]


def test_fp4_quantiser_bit_exact(ref):
    variant, d = ref
    for name in ("A", "B"):
        p, s = O.quant_fp4_ref32(d[f"fp4_{name}"], tie="ref_lut")
        assert (p == d[f"fp4_p{name}"]).all()           # includes every e2m1 tie point (row 0 of A)
        if variant == "ieee":
            assert (s == d[f"fp4_s{name}"]).all()
        else:                                            # fast-math division: scales within 2 ulp
            assert np.allclose(s, d[f"fp4_s{name}"], rtol=3e-7, atol=0)


def test_reference_ties_go_toward_zero(ref):
    _, d = ref
    nib = O.unpack_nibbles(d["fp4_pA"][:16])
    assert nib[:16].tolist() == [7, 0, 1, 2, 3, 4, 5, 6, 0, 9, 10, 11, 12, 13, 14, 0]


def test_restatement_bit_exact(ref, restatement):
    _, d = ref
    M, K = d["fp8_A"].shape
    N = d["fp8_B"].shape[1]
    qA, qB = np.ascontiguousarray(d["fp8_qA"]), np.ascontiguousarray(d["fp8_qB"])
    C = np.empty((M, N), np.float32)
    restatement.rs_fp8_gemm_per_tensor(vp(qA), vp(qB), vp(C), M, N, K, ctypes.c_float(d["fp8_scales"][0]),
                                       ctypes.c_float(d["fp8_scales"][1]))
    assert (C == d["fp8_C_per_tensor"]).all()
    sa, sb = np.ascontiguousarray(d["fp8_sa"]), np.ascontiguousarray(d["fp8_sb"])
    restatement.rs_fp8_gemm_groupwise(vp(qA), vp(qB), vp(C), M, N, K, 32, vp(sa), vp(sb))
    assert (C == d["fp8_C_groupwise"]).all()
    M, K = d["fp4_A"].shape
    N = d["fp4_B"].shape[1]
    C = np.empty((M, N), np.float32)
    restatement.rs_fp4_gemm(vp(np.ascontiguousarray(d["fp4_pA"])), vp(np.ascontiguousarray(d["fp4_pB"])), vp(C),
                            vp(np.ascontiguousarray(d["fp4_sA"])), vp(np.ascontiguousarray(d["fp4_sB"])), M, N, K)
    assert (C == d["fp4_C_nvfp4"]).all()
    assert (d["fp4_C_nvfp4"] == d["fp4_C_mxfp4"]).all()      # the reference's two "formats" are one


def test_restatement_quantisers_match_oracle(restatement):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(4096 * 9 + 7) * 2).astype(np.float32)
    x[64:96] = 0
    out, sc = np.empty(x.size, np.uint8), np.empty(1, np.float32)
    restatement.rs_quantize_fp8(vp(x), vp(out), vp(sc), ctypes.c_long(x.size))
    q, s = O.quant_fp8_per_tensor(x)
    assert (q == out).all() and s == sc[0]
    p, ss = np.empty((x.size + 1) // 2, np.uint8), np.empty((x.size + 31) // 32, np.float32)
    restatement.rs_quantize_fp4(vp(x), vp(p), vp(ss), ctypes.c_long(x.size))
    po, so = O.quant_fp4_ref32(x)
    assert (po == p).all() and (so == ss).all()


def test_gemm_oracle_vs_reference_cuda(ref):
    _, d = ref
    qA, qB_nk = d["fp8_qA"], np.ascontiguousarray(d["fp8_qB"].T)
    got = O.gemm_fp8_per_tensor(qA, qB_nk, d["fp8_scales"][0], d["fp8_scales"][1])
    assert rel_frobenius(got, d["fp8_C_per_tensor"]) < 1e-6
    got = O.gemm_fp8_groupwise(qA, qB_nk, d["fp8_sa"], d["fp8_sb"], group=32)
    assert rel_frobenius(got, d["fp8_C_groupwise"]) < 1e-6
    M, K = d["fp4_A"].shape
    N = d["fp4_B"].shape[1]
    got = O.gemm_fp4_ref32(d["fp4_pA"], d["fp4_sA"], d["fp4_pB"], d["fp4_sB"], M, N, K)
    assert rel_frobenius(got, d["fp4_C_nvfp4"]) < 1e-6
    A, B = d["grp_A"].astype(np.float64), d["grp_B"].astype(np.float64)
    assert rel_frobenius(d["grp_C_fixed"], np.einsum("gmk,gkn->gmn", A, B)) < 1e-6
    rows = d["grp_rows"]
    want = np.concatenate([A[g, :rows[g]] @ B[g] for g in range(len(rows))])
    assert rel_frobenius(d["grp_C_variable"], want) < 1e-6


def test_gemm_oracle_vs_reference_python_emulation():
    d = np.load(os.path.join(GOLDEN, "reference_py.npz"))
    got = O.gemm_fp8_per_tensor(d["fp8_qa"], np.ascontiguousarray(d["fp8_qb_kn"].T), d["fp8_sa"], d["fp8_sb"])
    assert rel_frobenius(got, d["fp8_c"]) < 1e-6
    a = (d["grp_a_bf16_bits"].astype(np.uint16).astype(np.uint32) << 16).view(np.float32)
    b = (d["grp_b_bf16_bits"].astype(np.uint16).astype(np.uint32) << 16).view(np.float32)
    want = np.einsum("gmk,gkn->gmn", a, b)
    assert rel_frobenius(d["grp_c"], want) < 1e-6


def test_block_scaled_oracles_are_self_consistent():
    rng = np.random.default_rng(9)
    a = rng.standard_normal((64, 256)).astype(np.float32)
    w = (rng.standard_normal((48, 256)) * 0.02).astype(np.float32)
    want = a @ w.T
    pa, sfa, gsa = O.quant_nvfp4(a)
    pb, sfb, gsb = O.quant_nvfp4(w)
    assert rel_frobenius(O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb), want) < 0.2
    pa, sfa = O.quant_mxfp4(a)
    pb, sfb = O.quant_mxfp4(w)
    assert rel_frobenius(O.gemm_mxfp4(pa, sfa, pb, sfb), want) < 0.25
    qa, sa = O.quant_fp8_groupwise(a)
    qb, sbb = O.quant_fp8_block(w)
    got = O.gemm_fp8_groupwise(qa, qb, sa, O.expand_block_scale(sbb, 48))
    assert rel_frobenius(got, want) < 0.06
