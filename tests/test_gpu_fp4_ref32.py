"""The reference's own FP4 container (fp32 scale per 32 flat elements, B packed [K, N/2]) on the GPU:
bit-exact against the outputs of the reference's CUDA kernels (tests/golden/reference_cuda_ieee.npz),
against the C restatement of those kernels and against the numpy oracle."""
import ctypes
import os

import numpy as np
import pytest
import torch

import dsl_tool_b200 as D
from oracle import quant_oracle as O
from tests.helpers import GOLDEN, rel_frobenius, vp

pytestmark = pytest.mark.gpu


def _dev(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def test_golden_quantiser_bit_exact(cuda_device):
    d = np.load(os.path.join(GOLDEN, "reference_cuda_ieee.npz"))
    for name in ("A", "B"):
        q, s = D.quantize_fp4_ref32(_dev(d[f"fp4_{name}"], cuda_device))
        assert (q.cpu().numpy() == d[f"fp4_p{name}"]).all()      # row 0 of A holds every e2m1 tie point
        assert (s.cpu().numpy() == d[f"fp4_s{name}"]).all()


def test_golden_gemm_bit_exact(cuda_device):
    d = np.load(os.path.join(GOLDEN, "reference_cuda_ieee.npz"))
    M, K = d["fp4_A"].shape
    N = d["fp4_B"].shape[1]
    pa = _dev(d["fp4_pA"].reshape(M, K // 2), cuda_device)
    pb = _dev(d["fp4_pB"].reshape(K, N // 2), cuda_device)
    sa = _dev(d["fp4_sA"].reshape(M, K // 32), cuda_device)
    sb = _dev(d["fp4_sB"].reshape(K // 32, N), cuda_device)
    for mx in (False, True):     # the reference's two "formats" are one (its tables are equal)
        c = D.fp4_gemm(pa, pb, scale_a=sa, scale_b=sb, use_mxfp4=mx, format="ref32")
        assert c.dtype == torch.float32 and tuple(c.shape) == (M, N)
        assert (c.cpu().numpy() == d["fp4_C_nvfp4"]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [1, 31, 32, 33, 4096 * 9 + 7, 1 << 20])
def test_quantiser_vs_oracle(cuda_device, dtype, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    if n > 96:
        x[64:96] = 0                      # an all-zero block: scale clamps to 1e-12, codes 0
        x[100] = -0.0
    xt = torch.from_numpy(x).to(dtype)
    q, s = D.quantize_fp4_ref32(xt.to(cuda_device))
    po, so = O.quant_fp4_ref32(xt.to(torch.float32).numpy())
    assert (q.cpu().numpy() == po).all()
    assert (s.cpu().numpy() == so).all()


@pytest.mark.parametrize("M,N,K", [(1, 8, 32), (7, 24, 96), (64, 64, 64), (65, 72, 160), (200, 328, 512), (512, 1024, 2048)])
def test_gemm_vs_restatement_bit_exact(cuda_device, restatement, M, N, K):
    rng = np.random.default_rng(M * 7 + N)
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    pa, sa_flat = O.quant_fp4_ref32(a)                     # blocks along K: scale_a [M, K/32]
    pbt, sbt = O.quant_fp4_ref32(np.ascontiguousarray(b.T))  # per (column, k-group) scales
    codes_kn = np.ascontiguousarray(O.unpack_nibbles(pbt).reshape(N, K).T)
    pb = O.pack_nibbles(codes_kn.reshape(-1))              # [K, N/2], pairs along N
    sb = np.ascontiguousarray(sbt.reshape(N, K // 32).T)   # [K/32, N]
    want = np.empty((M, N), np.float32)
    restatement.rs_fp4_gemm(vp(pa), vp(pb), vp(want), vp(sa_flat), vp(sb), M, N, K)
    got = D.fp4_gemm(_dev(pa.reshape(M, K // 2), cuda_device), _dev(pb.reshape(K, N // 2), cuda_device),
                     scale_a=_dev(sa_flat.reshape(M, K // 32), cuda_device), scale_b=_dev(sb, cuda_device),
                     format="ref32").cpu().numpy()
    assert (got == want).all()
    assert rel_frobenius(got, O.gemm_fp4_ref32(pa, sa_flat, pb, sb, M, N, K)) < 1e-6
    assert rel_frobenius(got, a @ b) < 0.2                 # and it is a GEMM of the inputs


def test_reference_flow_end_to_end(cuda_device, restatement):
    """quantise A and B flat, then multiply - the sequence of the reference's own driver (cuda/gemm/fp4_gemm.cu:180-191)."""
    rng = np.random.default_rng(5)
    M, N, K = 96, 128, 256
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    qa, sa = D.quantize_fp4_ref32(_dev(a, cuda_device))
    qb, sb = D.quantize_fp4_ref32(_dev(b, cuda_device))
    got = D.fp4_gemm(qa.view(M, K // 2), qb.view(K, N // 2), scale_a=sa.view(M, K // 32), scale_b=sb.view(K // 32, N),
                     format="ref32").cpu().numpy()
    pa, sa_o = O.quant_fp4_ref32(a)
    pb, sb_o = O.quant_fp4_ref32(b)
    want = np.empty((M, N), np.float32)
    restatement.rs_fp4_gemm(vp(pa), vp(pb), vp(want), vp(sa_o), vp(sb_o), M, N, K)
    assert (got == want).all()


def test_rejects_bad_shapes(cuda_device):
    pa = torch.zeros(4, 24, dtype=torch.uint8, device=cuda_device)      # K = 48: not a multiple of 32
    pb = torch.zeros(48, 4, dtype=torch.uint8, device=cuda_device)
    s = torch.ones(64, dtype=torch.float32, device=cuda_device)
    with pytest.raises(ValueError):
        D.fp4_gemm(pa, pb, scale_a=s, scale_b=s, format="ref32")
    with pytest.raises(ValueError):
        D.fp4_gemm(torch.zeros(4, 16, dtype=torch.uint8, device=cuda_device),
                   torch.zeros(32, 4, dtype=torch.uint8, device=cuda_device), format="ref32")
