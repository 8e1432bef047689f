"""GEMM kernels vs the oracle on the same seeded inputs.  GPU, through the C ABI.

Tolerance (north-star): relative Frobenius error <= 1e-3 on the fp32 result against the
fp32-accumulated dequantised oracle; the bf16 result is checked against the bf16-rounded oracle
(<= 1 bf16 ulp per element up to accumulation-order noise, relative Frobenius <= 4e-3)."""
import os

import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import (BF16_REL_FROB_TOL, GOLDEN, REL_FROB_TOL, activations, grouped_matmul, moe_offsets,
                           rel_frobenius, weights)

pytestmark = pytest.mark.gpu

MS = [1, 15, 16, 17, 127, 128, 129, 300]


def _status_ok():
    from dsl_tool_b200 import _lib
    _lib.check_status()


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("M", MS)
@pytest.mark.parametrize("N,K", [(256, 128), (520, 1040), (128, 512)])
def test_fp8_per_tensor(cuda_device, M, N, K):
    from dsl_tool_b200.gemm_kernels import gemm_fp8_quantized
    rng = np.random.default_rng(M * 7 + N)
    qa, sa = O.quant_fp8_per_tensor(activations(rng, M, K))
    qb, sb = O.quant_fp8_per_tensor(weights(rng, N, K))
    want = O.gemm_fp8_per_tensor(qa, qb, sa, sb)
    got = gemm_fp8_quantized(_t(qa), _t(qb), float(sa), float(sb), n=N)
    _status_ok()
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    got16 = gemm_fp8_quantized(_t(qa), _t(qb), float(sa), float(sb), n=N, out_dtype="bfloat16")
    assert got16.dtype == torch.bfloat16
    assert rel_frobenius(got16.float().cpu().numpy(), O.bf16_round(want)) <= BF16_REL_FROB_TOL
    assert torch.equal(got16, got.bfloat16())           # bf16 output is exactly the rounded fp32 output


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("M", MS)
@pytest.mark.parametrize("N,K", [(256, 256), (520, 1088), (128, 512), (72, 64)])
def test_fp4_block_scaled(cuda_device, fmt, M, N, K):
    from dsl_tool_b200.gemm_kernels import gemm_fp4_quantized
    rng = np.random.default_rng(M * 11 + N)
    a, w = activations(rng, M, K, outliers=True), weights(rng, N, K)
    if fmt == "nvfp4":
        pa, sfa, gsa = O.quant_nvfp4(a)
        pb, sfb, gsb = O.quant_nvfp4(w)
        want = O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)
    else:
        if K % 32:
            pytest.skip("K % 32")
        pa, sfa = O.quant_mxfp4(a)
        pb, sfb = O.quant_mxfp4(w)
        gsa = gsb = None
        want = O.gemm_mxfp4(pa, sfa, pb, sfb)
    got = gemm_fp4_quantized(_t(pa), _t(pb), _t(O.swizzle_sf(sfa)), _t(O.swizzle_sf(sfb)), format=fmt, n=N,
                             global_scale_a=None if gsa is None else float(gsa),
                             global_scale_b=None if gsb is None else float(gsb))
    _status_ok()
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL


@pytest.mark.parametrize("sb_block", [True, False])
@pytest.mark.parametrize("M", [1, 17, 128, 300])
@pytest.mark.parametrize("N,K", [(256, 256), (520, 1024), (100, 384)])
def test_fp8_groupwise(cuda_device, sb_block, M, N, K):
    from dsl_tool_b200.gemm_kernels import gemm_fp8_groupwise_quantized
    rng = np.random.default_rng(M * 13 + N)
    qa, sa = O.quant_fp8_groupwise(activations(rng, M, K))
    qb, sbb = O.quant_fp8_block(weights(rng, N, K))
    sb_col = O.expand_block_scale(sbb, N)                  # [K/128, N], the reference's layout
    want = O.gemm_fp8_groupwise(qa, qb, sa, sb_col)
    sb = _t(sbb[None]) if sb_block else _t(sb_col[None])
    got = gemm_fp8_groupwise_quantized(_t(qa), _t(qb), _t(sa), sb, n=N, sb_block=sb_block)
    _status_ok()
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL


@pytest.mark.parametrize("sb_block", [True, False])
@pytest.mark.parametrize("M,N", [(2560, 2000), (2304, 2304)])
def test_fp8_groupwise_last_round_cut_into_pieces(cuda_device, sb_block, M, N):
    """80 / 81 tiles of 256 x 256 on 74 CTA pairs: the tiles after the last full round run as 64-column pieces
    (also past a ragged right edge).  The pieces sum the same K groups in the same order, so besides matching the
    oracle the first 256 rows must equal, bit for bit, the same rows multiplied alone (8 / 9 tiles, nothing cut)."""
    from dsl_tool_b200.gemm_kernels import gemm_fp8_groupwise_quantized
    K = 384
    rng = np.random.default_rng(M + N)
    qa, sa = O.quant_fp8_groupwise(activations(rng, M, K))
    qb, sbb = O.quant_fp8_block(weights(rng, N, K))
    sb_col = O.expand_block_scale(sbb, N)
    want = O.gemm_fp8_groupwise(qa, qb, sa, sb_col)
    sb = _t(sbb[None]) if sb_block else _t(sb_col[None])
    got = gemm_fp8_groupwise_quantized(_t(qa), _t(qb), _t(sa), sb, n=N, sb_block=sb_block)
    _status_ok()
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    for r0 in (0, M - 256):
        alone = gemm_fp8_groupwise_quantized(_t(qa[r0:r0 + 256]), _t(qb), _t(sa[r0:r0 + 256]), sb, n=N, sb_block=sb_block)
        _status_ok()
        assert torch.equal(got[r0:r0 + 256], alone)


@pytest.mark.parametrize("group", [256, 384])
def test_fp8_groupwise_wider_groups_through_the_public_callable(cuda_device, group):
    """The reference's groupwise GEMM takes any group size (cuda/gemm/fp8_gemm.cu:110-116).  Multiples of 128 are served
    for already-quantised operands: one scale per `group` K-elements, [M, K/group] and [K/group, N], with B in the
    reference's [K, N] layout.  A group size below 128 (or not a multiple of it) is refused with a clear message."""
    from dsl_tool_b200 import fp8_gemm
    rng = np.random.default_rng(group)
    M, N, K = 300, 520, 768
    qa, sa = O.quant_fp8_groupwise(activations(rng, M, K), group=group)
    w = weights(rng, N, K)
    qb, sb_nk = O.quant_fp8_groupwise(w, group=group)            # per weight row and K group: [N, K/group]
    sb = np.ascontiguousarray(sb_nk.T)                             # the reference's [K/group, N]
    want = O.gemm_fp8_groupwise(qa, qb, sa, sb, group=group)
    got = fp8_gemm(_t(qa), _t(np.ascontiguousarray(qb.T)), _t(sa), _t(sb), mode="groupwise", group_size=group)
    _status_ok()
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    with pytest.raises(ValueError, match="multiple of 128"):
        fp8_gemm(_t(qa), _t(np.ascontiguousarray(qb.T)), _t(sa), _t(sb), mode="groupwise", group_size=32)


@pytest.mark.parametrize("gs", [20.0 / 2688.0, 3.0 / 2688.0])
def test_nvfp4_calibrated_activation_scale_is_one_pass_and_exact(cuda_device, gs):
    """`linear(..., act_global_scale=gs)`: the activations are quantised with the given global scale (no amax pass);
    bytes and product equal the oracle's with that scale - also when it is too small and values saturate."""
    from dsl_tool_b200 import pack_weight, quantize_fp4
    from dsl_tool_b200.gemm_kernels import linear
    rng = np.random.default_rng(91)
    M, N, K = 260, 384, 512
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()
    pw = pack_weight(w.cuda(), "nvfp4")
    got = linear(a.cuda(), pw, out_dtype="float32", act_global_scale=gs)
    _status_ok()
    pa, sfa, gsa = O.quant_nvfp4(a.float().numpy(), global_scale=np.float32(gs))
    pb, sfb, gsb = O.quant_nvfp4(w.float().numpy())
    assert rel_frobenius(got.cpu().numpy(), O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)) <= REL_FROB_TOL
    q, _, g = quantize_fp4(a.cuda(), "nvfp4", global_scale=gs)
    assert (q.cpu().numpy() == pa).all() and g.item() == np.float32(gs)
    assert torch.equal(got, linear(a.cuda(), pw, out_dtype="float32", act_global_scale=torch.tensor([gs], device="cuda")))


@pytest.mark.parametrize("M", [3, 100, 600])
def test_nvfp4_per_token_activation_scales_through_linear(cuda_device, M):
    """`linear(..., act_global_scale="per_token")` (decode, 1-CTA and CTA-pair kernels): the product equals the oracle's
    with per-token scales - (sum * weight global scale) * token scale - and the two-call form gives the same bits."""
    from dsl_tool_b200 import pack_weight, quantize_fp4
    from dsl_tool_b200.gemm_kernels import gemm_fp4_quantized, linear
    rng = np.random.default_rng(92 + M)
    N, K = 384, 1024
    a = torch.from_numpy(activations(rng, M, K, outliers=True) * rng.uniform(0.01, 30, (M, 1)).astype(np.float32)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()
    pw = pack_weight(w.cuda(), "nvfp4")
    got = linear(a.cuda(), pw, out_dtype="float32", act_global_scale="per_token")
    _status_ok()
    pa, sfa, gsa = O.quant_nvfp4(a.float().numpy(), "per_token")
    pb, sfb, gsb = O.quant_nvfp4(w.float().numpy())
    assert rel_frobenius(got.cpu().numpy(), O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)) <= REL_FROB_TOL
    q, sf, gs = quantize_fp4(a.cuda(), "nvfp4", global_scale="per_token")
    two = gemm_fp4_quantized(q, pw.q, sf, pw.scale, format="nvfp4", n=N, token_scale=gs, global_scale_b=pw.global_scale)
    assert torch.equal(two, got)
    with pytest.raises(ValueError, match="row_scale"):
        linear(a.cuda(), pw, act_global_scale="per_token", row_scale=torch.ones(M, device="cuda"))


def test_epilogue_row_and_column_rescale(cuda_device):
    from dsl_tool_b200.gemm_kernels import gemm_fp8_quantized
    rng = np.random.default_rng(5)
    M, N, K = 200, 328, 256
    qa, sa = O.quant_fp8_per_tensor(activations(rng, M, K))
    qb, sb = O.quant_fp8_per_tensor(weights(rng, N, K))
    rs = rng.uniform(0.5, 2, M).astype(np.float32)
    cs = rng.uniform(0.5, 2, N).astype(np.float32)
    want = O.gemm_fp8_per_tensor(qa, qb, sa, sb) * rs[:, None] * cs[None, :]
    got = gemm_fp8_quantized(_t(qa), _t(qb), _t(np.array([sa])), _t(np.array([sb])), n=N, row_scale=_t(rs), col_scale=_t(cs))
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL


def test_reference_golden_vectors_through_public_callables(cuda_device):
    """Inputs and outputs of the reference's own emulation (tests/golden) through fp8_gemm /
    grouped_gemm with the reference's positional arguments and [K,N] weight layout."""
    from dsl_tool_b200 import fp8_gemm, grouped_gemm
    d = np.load(os.path.join(GOLDEN, "reference_py.npz"))
    A = _t(d["fp8_qa"]).view(torch.float8_e4m3fn)
    B = _t(d["fp8_qb_kn"]).view(torch.float8_e4m3fn)
    got = fp8_gemm(A, B, float(d["fp8_sa"]), float(d["fp8_sb"]))
    assert got.dtype == torch.float32 and rel_frobenius(got.cpu().numpy(), d["fp8_c"]) <= 1e-5
    ga = _t(d["grp_a_bf16_bits"]).view(torch.bfloat16)
    gb = _t(d["grp_b_bf16_bits"]).view(torch.bfloat16)
    gc = grouped_gemm(ga, gb, 3)
    assert gc.dtype == torch.bfloat16 and gc.shape == (3, 70, 96)
    assert rel_frobenius(gc.float().cpu().numpy(), O.bf16_round(d["grp_c"])) <= BF16_REL_FROB_TOL
    gc32 = grouped_gemm(ga, gb, out_dtype="float32")
    assert rel_frobenius(gc32.cpu().numpy(), d["grp_c"]) <= 1e-5
    c = np.load(os.path.join(GOLDEN, "reference_cuda_ieee.npz"))
    got = fp8_gemm(_t(c["fp8_qA"]), _t(c["fp8_qB"]), float(c["fp8_scales"][0]), float(c["fp8_scales"][1]))
    assert rel_frobenius(got.cpu().numpy(), c["fp8_C_per_tensor"]) <= 1e-5
    got = grouped_gemm(_t(c["grp_A"]), _t(c["grp_B"]), 3, out_dtype="float32")
    assert rel_frobenius(got.cpu().numpy(), c["grp_C_fixed"]) <= 1e-2     # operands rounded to bf16


@pytest.mark.parametrize("fmt", ["fp8", "fp8_groupwise", "nvfp4", "mxfp4", "bf16"])
def test_quantise_then_gemm_matches_oracle_pipeline(cuda_device, fmt):
    """High-precision inputs through the public callables == oracle quantise + oracle GEMM."""
    from dsl_tool_b200 import fp4_gemm, fp8_gemm, grouped_gemm
    rng = np.random.default_rng(21)
    M, N, K = 200, 384, 512
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()              # K-major [N, K]
    ao, wo = a.float().numpy(), w.float().numpy()
    if fmt == "fp8":
        got = fp8_gemm(a.cuda(), w.cuda(), b_layout="nk")
        qa, sa = O.quant_fp8_per_tensor(ao); qb, sb = O.quant_fp8_per_tensor(wo)
        want = O.gemm_fp8_per_tensor(qa, qb, sa, sb)
        got_kn = fp8_gemm(a.cuda(), w.t().contiguous().cuda())        # the reference's B[K,N]
        assert torch.equal(got, got_kn)
    elif fmt == "fp8_groupwise":
        got = fp8_gemm(a.cuda(), w.cuda(), mode="groupwise", b_layout="nk")
        qa, sa = O.quant_fp8_groupwise(ao); qb, sbb = O.quant_fp8_block(wo)
        want = O.gemm_fp8_groupwise(qa, qb, sa, O.expand_block_scale(sbb, N))
    elif fmt == "nvfp4":
        got = fp4_gemm(a.cuda(), w.cuda(), b_layout="nk")
        want = O.gemm_nvfp4(*O.quant_nvfp4(ao), *O.quant_nvfp4(wo))
    elif fmt == "mxfp4":
        got = fp4_gemm(a.cuda(), w.cuda(), use_mxfp4=True, b_layout="nk")
        want = O.gemm_mxfp4(*O.quant_mxfp4(ao), *O.quant_mxfp4(wo))
    else:
        got = grouped_gemm(a.cuda()[None], w.cuda()[None], 1, b_layout="nk", out_dtype="float32")[0]
        want = ao @ wo.T
    _status_ok()
    assert rel_frobenius(got.float().cpu().numpy(), want) <= REL_FROB_TOL


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "fp8_groupwise", "fp8", "bf16"])
@pytest.mark.parametrize("skew", [0.0, 1.0])
def test_grouped_ragged_experts(cuda_device, fmt, skew):
    """MoE layout: routed rows sorted by expert, ragged (and, skewed, empty) groups."""
    from dsl_tool_b200 import grouped_gemm
    rng = np.random.default_rng(31)
    G, N, K = 16, 384, 512
    offs = moe_offsets(rng, 256, G, 4, bias_std=skew * 2.5)
    if skew:
        assert (np.diff(offs) == 0).any()                          # at least one empty expert
    M = int(offs[-1])
    a = torch.from_numpy(activations(rng, M, K)).bfloat16()
    w = torch.from_numpy(weights(rng, G * N, K).reshape(G, N, K)).bfloat16()
    ao, wo = a.float().numpy(), w.float().numpy()
    got = grouped_gemm(a.cuda(), w.cuda(), G, torch.from_numpy(offs).cuda(), format=fmt, b_layout="nk",
                       out_dtype="float32")
    _status_ok()
    flat = wo.reshape(G * N, K)
    if fmt == "nvfp4":
        pa, sfa, gsa = O.quant_nvfp4(ao); pb, sfb, gsb = O.quant_nvfp4(flat)
        A = O.dequant_fp4_values(pa, O.e4m3_decode(sfa), 16); B = O.dequant_fp4_values(pb, O.e4m3_decode(sfb), 16)
        want = grouped_matmul(A, B.reshape(G, N, K), offs) * np.float32(gsa * gsb)
    elif fmt == "mxfp4":
        pa, sfa = O.quant_mxfp4(ao); pb, sfb = O.quant_mxfp4(flat)
        A = O.dequant_fp4_values(pa, O.e8m0_decode(sfa), 32); B = O.dequant_fp4_values(pb, O.e8m0_decode(sfb), 32)
        want = grouped_matmul(A, B.reshape(G, N, K), offs)
    elif fmt == "fp8":
        qa, sa = O.quant_fp8_per_tensor(ao); qb, sb = O.quant_fp8_per_tensor(flat)
        want = grouped_matmul(O.e4m3_decode(qa), O.e4m3_decode(qb).reshape(G, N, K), offs) * sa * sb
    elif fmt == "fp8_groupwise":
        qa, sa = O.quant_fp8_groupwise(ao)
        want = np.zeros((M, N), np.float32)
        for g in range(G):
            r0, r1 = offs[g], offs[g + 1]
            if r1 > r0:
                qb, sbb = O.quant_fp8_block(wo[g])
                want[r0:r1] = O.gemm_fp8_groupwise(qa[r0:r1], qb, sa[r0:r1], O.expand_block_scale(sbb, N))
    else:
        want = grouped_matmul(ao, wo, offs)
    assert got.shape == (M, N)
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL


def test_grouped_fp8_groupwise_last_round_cut(cuda_device):
    """Row groups of 700, 0, 1300 and 290 rows = 3 + 0 + 6 + 2 row tiles x 8 column tiles = 88 tiles on 74 CTA pairs:
    the 14 tiles after the full round run as 64-column pieces, across group boundaries and ragged row tails.  Each
    group must match the oracle and equal, bit for bit, the same rows multiplied as a dense problem of their own."""
    from dsl_tool_b200 import grouped_gemm, fp8_gemm
    rng = np.random.default_rng(77)
    N, K = 2048, 384
    offs = np.array([0, 700, 700, 2000, 2290], np.int32)
    G, M = len(offs) - 1, int(offs[-1])
    a = torch.from_numpy(activations(rng, M, K)).bfloat16()
    w = torch.from_numpy(weights(rng, G * N, K).reshape(G, N, K)).bfloat16()
    ao, wo = a.float().numpy(), w.float().numpy()
    got = grouped_gemm(a.cuda(), w.cuda(), G, torch.from_numpy(offs).cuda(), format="fp8_groupwise", b_layout="nk",
                       out_dtype="float32")
    _status_ok()
    qa, sa = O.quant_fp8_groupwise(ao)
    for g in range(G):
        r0, r1 = int(offs[g]), int(offs[g + 1])
        if r1 == r0:
            continue
        qb, sbb = O.quant_fp8_block(wo[g])
        want = O.gemm_fp8_groupwise(qa[r0:r1], qb, sa[r0:r1], O.expand_block_scale(sbb, N))
        assert rel_frobenius(got[r0:r1].cpu().numpy(), want) <= REL_FROB_TOL
        alone = fp8_gemm(a[r0:r1].cuda(), w[g].cuda(), mode="groupwise", b_layout="nk")
        _status_ok()
        assert torch.equal(got[r0:r1], alone.float())


def test_run_to_run_determinism(cuda_device):
    from dsl_tool_b200 import fp4_gemm
    rng = np.random.default_rng(41)
    a = torch.from_numpy(activations(rng, 300, 1024)).bfloat16().cuda()
    w = torch.from_numpy(weights(rng, 520, 1024)).bfloat16().cuda()
    first = fp4_gemm(a, w, b_layout="nk")
    for _ in range(3):
        assert torch.equal(first, fp4_gemm(a, w, b_layout="nk"))


def test_output_canaries_untouched(cuda_device):
    """Rows / columns next to a ragged tile must not be written."""
    from dsl_tool_b200 import _lib
    from dsl_tool_b200.gemm_kernels import _epilogue
    import ctypes
    rng = np.random.default_rng(43)
    M, N, K, ldc = 130, 200, 256, 208
    qa, sa = O.quant_fp8_per_tensor(activations(rng, M, K))
    qb, sb = O.quant_fp8_per_tensor(weights(rng, N, K))
    A, B = _t(qa), _t(qb)
    buf = torch.full((M + 2, ldc), -777.0, device="cuda")
    keep = []
    ep = _epilogue(A.device, float(sa), float(sb), torch.float32, None, None, keep)
    rc = _lib.lib().dsl_gemm_fp8(A.data_ptr(), B.data_ptr(), buf[1:].data_ptr(), ldc, M, N, K, None, 1,
                                 ctypes.byref(ep), _lib.status_word(A.device).data_ptr(), _lib.stream_ptr())
    assert rc == 0
    out = buf.cpu().numpy()
    assert (out[0] == -777).all() and (out[-1] == -777).all() and (out[1:-1, N:] == -777).all()
    assert rel_frobenius(out[1:-1, :N], O.gemm_fp8_per_tensor(qa, qb, sa, sb)) <= REL_FROB_TOL


def test_argument_errors(cuda_device):
    from dsl_tool_b200 import fp4_gemm, fp8_gemm, grouped_gemm
    a = torch.randn(8, 64, device="cuda")
    with pytest.raises(ValueError, match="inner dimensions"):
        fp8_gemm(a, torch.randn(32, 8, device="cuda"))
    with pytest.raises(ValueError, match="mode must be"):
        fp8_gemm(a, torch.randn(64, 8, device="cuda"), mode="per_row")
    with pytest.raises(ValueError, match="scale_a and scale_b are required"):
        fp8_gemm(a.to(torch.float8_e4m3fn), torch.randn(64, 8, device="cuda").to(torch.float8_e4m3fn))
    with pytest.raises(ValueError, match="multiple of 32"):
        fp4_gemm(torch.randn(8, 48, device="cuda"), torch.randn(48, 8, device="cuda"))
    with pytest.raises(ValueError, match="num_groups=3"):
        grouped_gemm(torch.randn(2, 8, 64, device="cuda"), torch.randn(2, 64, 16, device="cuda"), 3)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fp8_gemm(torch.randn(8, 64), torch.randn(64, 8))


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "fp8", "bf16"])
@pytest.mark.parametrize("M", [1, 16, 100])
def test_decode_shapes_split_k(cuda_device, fmt, M):
    """Few rows and a long K: the GEMM is cut along K (fp32 partial sums in scratch, summed in
    slice order); results still match the oracle and are identical from run to run."""
    from dsl_tool_b200 import pack_weight
    from dsl_tool_b200.gemm_kernels import linear
    rng = np.random.default_rng(51 + M)
    N, K = 1024, 4096
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()
    ao, wo = a.float().numpy(), w.float().numpy()
    pw = pack_weight(w.cuda(), fmt)
    got = linear(a.cuda(), pw, out_dtype="float32")
    _status_ok()
    if fmt == "nvfp4":
        want = O.gemm_nvfp4(*O.quant_nvfp4(ao), *O.quant_nvfp4(wo))
    elif fmt == "mxfp4":
        want = O.gemm_mxfp4(*O.quant_mxfp4(ao), *O.quant_mxfp4(wo))
    elif fmt == "fp8":
        qa, sa = O.quant_fp8_per_tensor(ao); qb, sb = O.quant_fp8_per_tensor(wo)
        want = O.gemm_fp8_per_tensor(qa, qb, sa, sb)
    else:
        want = ao @ wo.T
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    assert torch.equal(got, linear(a.cuda(), pw, out_dtype="float32"))
    got16 = linear(a.cuda(), pw, out_dtype="bfloat16")
    assert torch.equal(got16, got.bfloat16())
