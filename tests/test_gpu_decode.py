"""The weight-streaming kernel for decode shapes (at most 128 activation rows, one row group; beyond
32 rows only where the cluster combine applies, else the tiled split-K kernel, covered by the same
cases): operand roles swapped, K cut into runs whose fp32 partial tiles are summed in ascending K
order - inside a thread-block cluster through shared memory when a tile has 2 or 4 runs, through
scratch otherwise.
Same oracle and tolerance as the tiled kernels (relative Frobenius <= 1e-3 on the fp32 result)."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import REL_FROB_TOL, activations, rel_frobenius, weights

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _oracle(fmt, ao, wo):
    if fmt == "nvfp4":
        return O.gemm_nvfp4(*O.quant_nvfp4(ao), *O.quant_nvfp4(wo))
    if fmt == "mxfp4":
        return O.gemm_mxfp4(*O.quant_mxfp4(ao), *O.quant_mxfp4(wo))
    if fmt == "fp8":
        qa, sa = O.quant_fp8_per_tensor(ao)
        qb, sb = O.quant_fp8_per_tensor(wo)
        return O.gemm_fp8_per_tensor(qa, qb, sa, sb)
    return ao @ wo.T


# every token bucket of the streaming kernel (16 / 32 / 64 / 128 accumulator columns) and both sides of each boundary
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "fp8", "bf16"])
@pytest.mark.parametrize("M", [1, 16, 17, 32, 33, 64, 65, 128])
def test_token_buckets(cuda_device, fmt, M):
    from dsl_tool_b200 import _lib, pack_weight
    from dsl_tool_b200.gemm_kernels import linear
    rng = np.random.default_rng(900 + M)
    N, K = 2304, 3072          # 18 column tiles; tile runs are shared between CTAs
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()
    pw = pack_weight(w.cuda(), fmt)
    got = linear(a.cuda(), pw, out_dtype="float32")
    _lib.check_status()
    assert rel_frobenius(got.cpu().numpy(), _oracle(fmt, a.float().numpy(), w.float().numpy())) <= REL_FROB_TOL
    assert torch.equal(got, linear(a.cuda(), pw, out_dtype="float32"))          # run-to-run identical
    assert torch.equal(linear(a.cuda(), pw, out_dtype="bfloat16"), got.bfloat16())


# ragged edges: N not a multiple of 128, K not a multiple of one 128-byte stage
@pytest.mark.parametrize("fmt,N,K", [("nvfp4", 1000, 2080), ("mxfp4", 1160, 2080), ("fp8", 1000, 2064), ("bf16", 392, 1032),
                                     ("nvfp4", 128, 8192), ("fp8", 8200, 512)])
@pytest.mark.parametrize("M", [3, 48])
def test_ragged_edges(cuda_device, fmt, N, K, M):
    from dsl_tool_b200 import _lib, pack_weight
    from dsl_tool_b200.gemm_kernels import linear
    rng = np.random.default_rng(N + K + M)
    a = torch.from_numpy(activations(rng, M, K)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()
    got = linear(a.cuda(), pack_weight(w.cuda(), fmt), out_dtype="float32")
    _lib.check_status()
    assert rel_frobenius(got.cpu().numpy(), _oracle(fmt, a.float().numpy(), w.float().numpy())) <= REL_FROB_TOL


# one case per way of cutting the work: clusters of 4 and of 2 runs per tile, whole tiles (no cut),
# and runs that cross tile borders (more column tiles than SMs)
@pytest.mark.parametrize("fmt", ["nvfp4", "fp8"])
@pytest.mark.parametrize("N,K,M", [(2304, 4096, 16), (6400, 4096, 9), (12800, 1024, 16), (19200, 2048, 5), (19200, 2048, 30),
                                   (2304, 4096, 64), (6400, 4096, 128), (19200, 2048, 100)])
def test_work_split_modes(cuda_device, fmt, N, K, M):
    from dsl_tool_b200 import _lib, pack_weight
    from dsl_tool_b200.gemm_kernels import linear
    rng = np.random.default_rng(N + M)
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16()
    w = torch.from_numpy(weights(rng, N, K)).bfloat16()
    pw = pack_weight(w.cuda(), fmt)
    got = linear(a.cuda(), pw, out_dtype="float32")
    _lib.check_status()
    assert rel_frobenius(got.cpu().numpy(), _oracle(fmt, a.float().numpy(), w.float().numpy())) <= REL_FROB_TOL
    for _ in range(3):
        assert torch.equal(got, linear(a.cuda(), pw, out_dtype="float32"))      # whoever arrives last, same sum


def test_same_numbers_as_the_tiled_kernel(cuda_device):
    """An exactly representable problem (small integers, power-of-two scales): the result does not
    depend on summation order, so the streamed path must equal the exact integer product."""
    from dsl_tool_b200.gemm_kernels import gemm_fp8_quantized
    rng = np.random.default_rng(77)
    M, N, K = 24, 1536, 4096
    ai = rng.integers(-4, 5, (M, K)).astype(np.float32)
    wi = rng.integers(-4, 5, (N, K)).astype(np.float32)
    qa, qb = O.e4m3_encode(ai), O.e4m3_encode(wi)
    got = gemm_fp8_quantized(_t(qa), _t(qb), 0.5, 0.25, n=N)
    assert np.array_equal(got.cpu().numpy(), (ai @ wi.T) * 0.125)


def test_epilogue_scales_and_strided_output(cuda_device):
    from dsl_tool_b200.gemm_kernels import gemm_fp8_quantized
    rng = np.random.default_rng(78)
    M, N, K = 20, 1100, 2048
    qa, sa = O.quant_fp8_per_tensor(activations(rng, M, K))
    qb, sb = O.quant_fp8_per_tensor(weights(rng, N, K))
    rs = rng.uniform(0.5, 2, M).astype(np.float32)
    cs = rng.uniform(0.5, 2, N).astype(np.float32)
    want = O.gemm_fp8_per_tensor(qa, qb, sa, sb) * rs[:, None] * cs[None, :]
    got = gemm_fp8_quantized(_t(qa), _t(qb), _t(np.array([sa])), _t(np.array([sb])), n=N, row_scale=_t(rs), col_scale=_t(cs))
    assert rel_frobenius(got.cpu().numpy(), want) <= REL_FROB_TOL
    got16 = gemm_fp8_quantized(_t(qa), _t(qb), float(sa), float(sb), n=N, row_scale=_t(rs), col_scale=_t(cs),
                               out_dtype="bfloat16")
    assert torch.equal(got16, got.bfloat16())
