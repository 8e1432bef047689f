"""The benchmark configurations at their full sizes on the GPU.  The oracle cannot multiply these sizes
in seconds, so the checks are (a) exact parity on a sample of output rows, whose oracle needs only
those activation rows against the full weight, (b) bit-exact quantised bytes on the same rows, and
(c) a closed-form case that covers every tile: constant rows times constant rows."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import REL_FROB_TOL, moe_offsets, rel_frobenius

pytestmark = pytest.mark.gpu


def _gen(shape, std, seed, outliers=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda") * std
    if outliers:
        mask = torch.rand(shape, generator=g, device="cuda") < 1e-3
        x = torch.where(mask, torch.where(torch.rand(shape, generator=g, device="cuda") < 0.5, -20.0, 20.0), x)
    return x.bfloat16()


def _rows(m, count, seed):
    r = np.random.default_rng(seed).choice(m, size=min(count, m), replace=False)
    r[:3] = [0, m // 2, m - 1][: len(r[:3])]
    return np.sort(np.unique(r))


def test_nvfp4_8192_cubed_sampled_rows(cuda_device):
    from dsl_tool_b200 import fp4_gemm, quantize_fp4
    M = N = K = 8192
    a, w = _gen((M, K), 1.0, 1, outliers=True), _gen((N, K), 0.02, 2)
    got = fp4_gemm(a, w, b_layout="nk")
    rows = _rows(M, 24, 3)
    ao, wo = a.float().cpu().numpy(), w.float().cpu().numpy()
    gsa = O.nvfp4_global_scale(ao)
    pa, sfa, _ = O.quant_nvfp4(ao[rows], global_scale=gsa)      # the block rule is row-local given the global scale
    pb, sfb, gsb = O.quant_nvfp4(wo)
    want = O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)
    assert rel_frobenius(got[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= REL_FROB_TOL
    q, sf, gs = quantize_fp4(a, "nvfp4")
    assert gs.item() == gsa and (q[torch.from_numpy(rows).cuda()].cpu().numpy() == pa).all()
    assert (O.unswizzle_sf(sf.cpu().numpy(), M, K // 16)[rows] == sfa).all()


def test_mxfp4_llama70b_up_sampled_rows(cuda_device):
    from dsl_tool_b200 import fp4_gemm
    M, K, N = 8192, 8192, 28672
    a, w = _gen((M, K), 1.0, 4), _gen((N, K), 0.015, 5)
    got = fp4_gemm(a, w, use_mxfp4=True, b_layout="nk", out_dtype="bfloat16")
    rows = _rows(M, 8, 6)
    pa, sfa = O.quant_mxfp4(a[torch.from_numpy(rows).cuda()].float().cpu().numpy())
    pb, sfb = O.quant_mxfp4(w.float().cpu().numpy())
    want = O.bf16_round(O.gemm_mxfp4(pa, sfa, pb, sfb))
    assert rel_frobenius(got[torch.from_numpy(rows).cuda()].float().cpu().numpy(), want) <= 4e-3


def test_fp8_groupwise_llama8b_mlp_sampled_rows(cuda_device):
    from dsl_tool_b200 import fp8_gemm
    M, K, N = 4096, 4096, 14336
    a, w = _gen((M, K), 1.0, 7), _gen((N, K), 0.02, 8)
    got = fp8_gemm(a, w, mode="groupwise", b_layout="nk")
    rows = _rows(M, 24, 9)
    qa, sa = O.quant_fp8_groupwise(a[torch.from_numpy(rows).cuda()].float().cpu().numpy())
    qb, sbb = O.quant_fp8_block(w.float().cpu().numpy())
    want = O.gemm_fp8_groupwise(qa, qb, sa, O.expand_block_scale(sbb, N))
    assert rel_frobenius(got[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= REL_FROB_TOL


def test_moe_layer_literal_config_sampled_rows(cuda_device):
    """64 experts, 16384 tokens routed top-8 (131072 rows), K=4096, N=2x1536, NVFP4."""
    from dsl_tool_b200 import grouped_gemm
    rng = np.random.default_rng(10)
    G, K, N = 64, 4096, 3072
    offs = moe_offsets(rng, 16384, G, 8)
    M = int(offs[-1])
    assert M == 131072
    a, w = _gen((M, K), 1.0, 11), _gen((G, N, K), 0.02, 12)
    got = grouped_gemm(a, w, G, torch.from_numpy(offs).cuda(), format="nvfp4", b_layout="nk", out_dtype="float32")
    ao_amax = float(a.float().abs().max().item())
    gsa = np.float32(np.float32(ao_amax) / np.float32(2688.0))
    wo = w.float().cpu().numpy().reshape(G * N, K)
    pb, sfb, gsb = O.quant_nvfp4(wo)
    B = O.dequant_fp4_values(pb, O.e4m3_decode(sfb), 16).reshape(G, N, K)
    for g in (0, 17, 63):
        r0, r1 = int(offs[g]), int(offs[g + 1])
        rows = np.unique(np.concatenate([[r0, r1 - 1], rng.integers(r0, r1, 6)]))
        pa, sfa, _ = O.quant_nvfp4(a[torch.from_numpy(rows).cuda()].float().cpu().numpy(), global_scale=gsa)
        A = O.dequant_fp4_values(pa, O.e4m3_decode(sfa), 16)
        want = (A @ B[g].T) * np.float32(gsa * gsb)
        assert rel_frobenius(got[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= REL_FROB_TOL


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "fp8", "fp8_groupwise"])
def test_every_tile_closed_form(cuda_device, fmt):
    """A[m,:] = r_m, W[n,:] = c_n with r, c on the e2m1 grid: every format stores them exactly, so
    C[m,n] = K * r_m * c_n exactly (sums of equal products stay exact in fp32 here).  A missed,
    duplicated or misplaced tile anywhere in the 4096 x 8192 output shows up."""
    from dsl_tool_b200 import fp4_gemm, fp8_gemm
    M, N, K = 4096 + 37, 8192, 2048
    rv = torch.tensor([0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -1.0], device="cuda")
    r = rv[torch.arange(M, device="cuda") % 8]
    c = rv[(torch.arange(N, device="cuda") * 5 + 3) % 8]
    r[0], c[0] = 6.0, 6.0                                   # pins every amax-derived scale
    a = r[:, None].expand(M, K).contiguous().bfloat16()
    w = c[:, None].expand(N, K).contiguous().bfloat16()
    if fmt == "nvfp4":
        got = fp4_gemm(a, w, b_layout="nk")
    elif fmt == "mxfp4":
        got = fp4_gemm(a, w, use_mxfp4=True, b_layout="nk")
    elif fmt == "fp8":
        got = fp8_gemm(a, w, b_layout="nk")
    else:
        got = fp8_gemm(a, w, mode="groupwise", b_layout="nk")
    want = (K * r[:, None] * c[None, :]).float()
    if fmt in ("mxfp4",):
        assert torch.equal(got, want)
    else:       # scales that are not powers of two round once; the structure check is what matters
        assert float((got - want).norm() / want.norm()) <= 5e-2
        assert float(((got - want).abs() / want.abs()).max()) <= 0.1
