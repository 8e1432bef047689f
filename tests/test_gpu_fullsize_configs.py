"""The benchmark configurations that the other full-size file does not reach, at their stated sizes:

  * NVFP4, N = K = 8192 with 0.1 % outliers at 20 sigma, M = 1 / 16 / 128 (weight-streaming kernel with 16- and
    128-token accumulators, partial tiles combined inside clusters) and M = 1024 (CTA-pair kernel),
  * MXFP4 at the Llama-3-70B down-projection shape (M = 8192, K = 28672, N = 8192),
  * the MoE gate/up GEMM (64 experts, 131072 routed rows, K = 4096, N = 3072) with FP8 group scales,
  * the same MoE GEMM in NVFP4 under skewed routing (one expert with no rows, one with several thousand).

Where the oracle cannot multiply the whole problem in seconds it is evaluated on sampled activation rows
(quantisation is row-local once the global scale is known) and, for the largest weight, on sampled weight rows
(MXFP4 and the 128 x 128 FP8 blocks are local to rows / row blocks).  Quantised bytes are compared bit for bit,
products within the relative-Frobenius bound of 1e-3 on the fp32 result."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import REL_FROB_TOL, rel_frobenius

pytestmark = pytest.mark.gpu


def _gen(shape, std, seed, outliers=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda") * std
    if outliers:
        mask = torch.rand(shape, generator=g, device="cuda") < 1e-3
        x = torch.where(mask, torch.where(torch.rand(shape, generator=g, device="cuda") < 0.5, -20.0, 20.0), x)
    return x.bfloat16()


def _idx(rows):
    return torch.from_numpy(np.asarray(rows)).cuda()


def _sample(m, count, seed):
    r = np.random.default_rng(seed).choice(m, size=min(count, m), replace=False)
    return np.unique(np.concatenate([[0, m - 1], r]))


@pytest.fixture(scope="module")
def nvfp4_weight_8192():
    """The 8192 x 8192 N(0, 0.02) weight: device tensor, packed form, and the oracle's quantised form."""
    from dsl_tool_b200 import pack_weight
    w = _gen((8192, 8192), 0.02, 2)
    pb, sfb, gsb = O.quant_nvfp4(w.float().cpu().numpy())
    return pack_weight(w, "nvfp4"), (pb, sfb, gsb)


@pytest.mark.parametrize("M", [1, 16, 128, 1024])
def test_nvfp4_n8192_k8192_decode_to_prefill(cuda_device, nvfp4_weight_8192, M):
    from dsl_tool_b200 import _lib, fp4_gemm, quantize_fp4
    pw, (pb, sfb, gsb) = nvfp4_weight_8192
    K = 8192
    a = _gen((M, K), 1.0, 100 + M, outliers=True)
    got = fp4_gemm(a, pw)
    _lib.check_status()
    ao = a.float().cpu().numpy()
    rows = np.arange(M) if M <= 128 else _sample(M, 48, 5)
    gsa = O.nvfp4_global_scale(ao)
    pa, sfa, _ = O.quant_nvfp4(ao[rows], global_scale=gsa)
    want = O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)
    assert rel_frobenius(got[_idx(rows)].cpu().numpy(), want) <= REL_FROB_TOL
    q, sf, gs = quantize_fp4(a, "nvfp4")
    assert gs.item() == gsa and (q[_idx(rows)].cpu().numpy() == pa).all()
    assert (O.unswizzle_sf(sf.cpu().numpy(), M, K // 16)[rows] == sfa).all()
    assert torch.equal(fp4_gemm(a, pw, out_dtype="bfloat16"), got.bfloat16())
    assert torch.equal(fp4_gemm(a, pw), got)                                    # run-to-run identical


def test_mxfp4_llama70b_down_sampled_rows_and_columns(cuda_device):
    from dsl_tool_b200 import _lib, fp4_gemm
    M, K, N = 8192, 28672, 8192
    a, w = _gen((M, K), 1.0, 21), _gen((N, K), 0.015, 22)
    got = fp4_gemm(a, w, use_mxfp4=True, b_layout="nk")
    _lib.check_status()
    rows, cols = _sample(M, 30, 23), _sample(N, 600, 24)
    pa, sfa = O.quant_mxfp4(a[_idx(rows)].float().cpu().numpy())
    pb, sfb = O.quant_mxfp4(w[_idx(cols)].float().cpu().numpy())
    want = O.gemm_mxfp4(pa, sfa, pb, sfb)
    sub = got[_idx(rows)][:, _idx(cols)].cpu().numpy()
    assert rel_frobenius(sub, want) <= REL_FROB_TOL


def _routing(tokens, experts, topk, seed, bias=None):
    rng = np.random.default_rng(seed)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    if bias is not None:
        logits += bias[None, :]
    top = np.argpartition(-logits, topk - 1, axis=1)[:, :topk]
    counts = np.bincount(top.reshape(-1), minlength=experts)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def test_moe_fp8_groupwise_literal_config_sampled_rows(cuda_device):
    from dsl_tool_b200 import _lib, grouped_gemm
    G, K, N = 64, 4096, 3072
    offs = _routing(16384, G, 8, 31)
    M = int(offs[-1])
    assert M == 131072
    a, w = _gen((M, K), 1.0, 32), _gen((G, N, K), 0.02, 33)
    got = grouped_gemm(a, w, G, torch.from_numpy(offs).cuda(), format="fp8_groupwise", b_layout="nk", out_dtype="float32")
    _lib.check_status()
    rng = np.random.default_rng(34)
    for g in (0, 29, 63):
        r0, r1 = int(offs[g]), int(offs[g + 1])
        rows = np.unique(np.concatenate([[r0, r1 - 1], rng.integers(r0, r1, 10)]))
        qa, sa = O.quant_fp8_groupwise(a[_idx(rows)].float().cpu().numpy())
        qb, sbb = O.quant_fp8_block(w[g].float().cpu().numpy())
        want = O.gemm_fp8_groupwise(qa, qb, sa, O.expand_block_scale(sbb, N))
        assert rel_frobenius(got[_idx(rows)].cpu().numpy(), want) <= REL_FROB_TOL


def test_moe_nvfp4_skewed_routing_empty_and_oversized_experts(cuda_device):
    from dsl_tool_b200 import _lib, grouped_gemm, quantize_fp4
    G, K, N = 64, 4096, 3072
    bias = (np.random.default_rng(41).standard_normal(G) * 0.6).astype(np.float32)
    bias[5] = -1e9                                                  # an expert nobody is routed to
    offs = _routing(16384, G, 8, 42, bias)
    counts = np.diff(offs)
    M = int(offs[-1])
    assert M == 131072 and counts[5] == 0 and counts.max() > 5000 and counts[counts > 0].min() < 300
    a, w = _gen((M, K), 1.0, 43), _gen((G, N, K), 0.02, 44)
    offs_dev = torch.from_numpy(offs).cuda()
    got = grouped_gemm(a, w, G, offs_dev, format="nvfp4", b_layout="nk", out_dtype="float32")
    _lib.check_status()
    gsa = np.float32(np.float32(a.float().abs().max().item()) / np.float32(2688.0))
    gsb = np.float32(np.float32(w.float().abs().max().item()) / np.float32(2688.0))   # one global scale for all experts
    q, _, gs = quantize_fp4(a, "nvfp4", group_offsets=offs_dev)
    assert gs.item() == gsa
    rng = np.random.default_rng(45)
    big, small = int(np.argmax(counts)), int(np.argmin(np.where(counts > 0, counts, 1 << 30)))
    for g in (big, small, 4, 6, 63):                                # 4 and 6: the neighbours of the empty expert
        r0, r1 = int(offs[g]), int(offs[g + 1])
        rows = np.unique(np.concatenate([[r0, r1 - 1], rng.integers(r0, r1, 8)]))
        pa, sfa, _ = O.quant_nvfp4(a[_idx(rows)].float().cpu().numpy(), global_scale=gsa)
        assert (q[_idx(rows)].cpu().numpy() == pa).all()
        pb, sfb, _ = O.quant_nvfp4(w[g].float().cpu().numpy(), global_scale=gsb)   # block scales are row-local
        assert rel_frobenius(got[_idx(rows)].cpu().numpy(), O.gemm_nvfp4(pa, sfa, gsa, pb, sfb, gsb)) <= REL_FROB_TOL
