"""Fused SwiGLU epilogue: the GEMM of a fused gate/up projection writes silu(gate) * up ([M, N/2])
instead of the [M, N] projection (the consumer in the reference is swiglu on [B, 2H],
cuda/activations/fused_gated_activations.cu:75-90, silu(x) = x / (1 + exp(-x)) at :27-29).
Oracle: the oracle GEMM on the same quantised operands, then the reference's formula in fp32."""
import numpy as np
import pytest
import torch

import dsl_tool_b200 as D
from oracle import quant_oracle as O
from tests.helpers import BF16_REL_FROB_TOL, REL_FROB_TOL, activations, moe_offsets, rel_frobenius, weights

pytestmark = pytest.mark.gpu


_interleave = O.interleave_gate_up


def _oracle_gemm(fmt, ao, wo):
    n = wo.shape[0]
    if fmt == "nvfp4":
        return O.gemm_nvfp4(*O.quant_nvfp4(ao), *O.quant_nvfp4(wo))
    if fmt == "mxfp4":
        return O.gemm_mxfp4(*O.quant_mxfp4(ao), *O.quant_mxfp4(wo))
    if fmt == "fp8":
        qa, sa = O.quant_fp8_per_tensor(ao)
        qb, sb = O.quant_fp8_per_tensor(wo)
        return O.gemm_fp8_per_tensor(qa, qb, sa, sb)
    if fmt == "fp8_block128":
        qa, sa = O.quant_fp8_groupwise(ao)
        qb, sbb = O.quant_fp8_block(wo)
        return O.gemm_fp8_groupwise(qa, qb, sa, O.expand_block_scale(sbb, n))
    return ao @ wo.T


_swiglu_of_interleaved = lambda full: O.gated_of_interleaved(full, "swiglu")
_geglu_of_interleaved = lambda full: O.gated_of_interleaved(full, "geglu")


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8_block128", "bf16"])
@pytest.mark.parametrize("M", [5, 300])
def test_dense_geglu(cuda_device, fmt, M):
    rng = np.random.default_rng(M)
    H, K = 192, 512
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, 2 * H, K, std=0.05)).bfloat16()
    pw = D.pack_weight(w.cuda(), fmt, gate_up_interleave=True)
    got = D.linear(a.cuda(), pw, activation="geglu")
    want = _geglu_of_interleaved(_oracle_gemm(fmt, a.float().numpy(), _interleave(w.float().numpy())))
    assert tuple(got.shape) == (M, H) and rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "fp8", "fp8_block128", "bf16"])
@pytest.mark.parametrize("M,H", [(5, 192), (300, 192), (77, 100), (300, 328)])
def test_dense_swiglu(cuda_device, fmt, M, H):
    rng = np.random.default_rng(M + H)
    K = 512
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, 2 * H, K, std=0.05)).bfloat16()       # [gate; up] rows
    pw = D.pack_weight(w.cuda(), fmt, gate_up_interleave=True)
    assert pw.gate_up_interleaved and pw.n == 2 * H
    got = D.linear(a.cuda(), pw, activation="swiglu")
    assert tuple(got.shape) == (M, H) and got.dtype == torch.float32
    want = _swiglu_of_interleaved(_oracle_gemm(fmt, a.float().numpy(), _interleave(w.float().numpy())))
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    got16 = D.linear(a.cuda(), pw, activation="swiglu", out_dtype="bfloat16")
    assert torch.equal(got16, got.bfloat16())
    # and it is the unfused sequence: projection, then the reference's activation on [gate | up]
    proj = D.linear(a.cuda(), D.pack_weight(w.cuda(), fmt)).cpu().numpy()
    if fmt != "fp8_block128":          # 128-row weight blocks see other rows once the rows are interleaved
        g, u = proj[:, :H], proj[:, H:]
        assert rel_frobenius(got.cpu().numpy(), (g / (1 + np.exp(-g))) * u) <= 1e-5


def test_groupwise_swiglu_with_the_last_round_cut(cuda_device):
    """2560 x 2048 gate/up columns = 80 tiles on 74 CTA pairs: the tiles after the full round run as 64-column
    pieces, i.e. 32 (gate, up) pairs each, through the activation epilogue of the group-scaled FP8 kernel."""
    rng = np.random.default_rng(2560)
    M, H, K = 2560, 1024, 256
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, 2 * H, K, std=0.05)).bfloat16()
    pw = D.pack_weight(w.cuda(), "fp8_block128", gate_up_interleave=True)
    got = D.linear(a.cuda(), pw, activation="swiglu")
    want = _swiglu_of_interleaved(_oracle_gemm("fp8_block128", a.float().numpy(), _interleave(w.float().numpy())))
    assert tuple(got.shape) == (M, H) and rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    alone = D.linear(a[-256:].cuda(), pw, activation="swiglu")             # 8 tiles, nothing cut: the same bits
    assert torch.equal(got[-256:], alone)


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8_groupwise", "bf16"])
def test_grouped_swiglu_ragged_experts(cuda_device, fmt):
    rng = np.random.default_rng(12)
    G, K, H = 6, 256, 128
    offs = moe_offsets(rng, 96, G, 4, bias_std=1.0)
    offs[3] = offs[2]                                   # an empty expert
    M = int(offs[-1])
    a = torch.from_numpy(activations(rng, M, K)).bfloat16()
    w = torch.from_numpy((rng.standard_normal((G, 2 * H, K)) * 0.05).astype(np.float32)).bfloat16()   # [G, 2H, K]
    got = D.grouped_gemm(a.cuda(), w.cuda(), expert_offsets=torch.from_numpy(offs).cuda(), format=fmt, b_layout="nk",
                         activation="swiglu", out_dtype="float32")
    assert tuple(got.shape) == (M, H)
    ofmt = {"fp8_groupwise": "fp8_block128"}.get(fmt, fmt)
    wi = _interleave(w.float().numpy())
    ao = a.float().numpy()
    want = np.zeros((M, H), np.float32)
    if fmt == "nvfp4":                                   # one global scale over all experts, as pack_weight derives it
        pa, sfa, gsa = O.quant_nvfp4(ao)
        gsb = O.nvfp4_global_scale(wi)
    for g in range(G):
        r0, r1 = int(offs[g]), int(offs[g + 1])
        if r1 == r0:
            continue
        if fmt == "nvfp4":
            pb, sfb, _ = O.quant_nvfp4(wi[g], global_scale=gsb)
            full = O.gemm_nvfp4(pa[r0:r1], sfa[r0:r1], gsa, pb, sfb, gsb)
        else:
            full = _oracle_gemm(ofmt, ao[r0:r1], wi[g])
        want[r0:r1] = _swiglu_of_interleaved(full)
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL


def test_argument_checks(cuda_device):
    a = torch.randn(8, 256, device=cuda_device)
    w = torch.randn(128, 256, device=cuda_device)
    with pytest.raises(ValueError):
        D.linear(a, D.pack_weight(w, "fp8"), activation="swiglu")            # not packed for it
    with pytest.raises(ValueError):
        D.linear(a, D.pack_weight(w, "fp8", gate_up_interleave=True), activation="gelu")
    with pytest.raises(ValueError):
        D.pack_weight(torch.randn(127, 256, device=cuda_device), "fp8", gate_up_interleave=True)
