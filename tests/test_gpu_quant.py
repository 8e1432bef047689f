"""Quantise / scale-pack kernels vs the oracle: bytes must be identical.  GPU, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import activations, weights

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]
SHAPES = [(1, 32), (7, 96), (128, 256), (129, 1056), (300, 512), (1024, 1024), (1024, 4096)]


def _inputs(shape, dtype, seed, outliers=True):
    rng = np.random.default_rng(seed)
    x = activations(rng, *shape, outliers=outliers)
    if shape[0] > 3:
        x[3, :] = 0.0                                   # an all-zero row
    x[0, :16] = np.array([6, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5, -0.0],
                         np.float32)[: min(16, shape[1])]
    xt = torch.from_numpy(x).to(dtype)
    return xt.cuda(), xt.float().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_fp8_modes(cuda_device, shape, dtype):
    from dsl_tool_b200 import quantize_fp8
    xc, xo = _inputs(shape, dtype, 1)
    q, s = quantize_fp8(xc, "per_tensor")
    qo, so = O.quant_fp8_per_tensor(xo)
    assert s.item() == so and (q.cpu().numpy() == qo).all()
    q, s = quantize_fp8(xc, "per_tensor", scale=0.037)                 # static scale
    qo, _ = O.quant_fp8_per_tensor(xo, scale=np.float32(0.037))
    assert (q.cpu().numpy() == qo).all() and s.item() == np.float32(0.037)
    if shape[1] % 16 == 0:
        q, s = quantize_fp8(xc, "groupwise")
        qo, so = O.quant_fp8_groupwise(xo)
        assert (s.cpu().numpy() == so).all() and (q.cpu().numpy() == qo).all()
        q, s = quantize_fp8(xc, "block128")
        qo, so = O.quant_fp8_block(xo)
        assert (s.cpu().numpy() == so).all() and (q.cpu().numpy() == qo).all()


def test_fp8_per_tensor_odd_length(cuda_device):
    from dsl_tool_b200 import quantize_fp8
    xc, xo = _inputs((5, 37), torch.float32, 2)
    q, s = quantize_fp8(xc, "per_tensor")
    qo, so = O.quant_fp8_per_tensor(xo)
    assert s.item() == so and (q.cpu().numpy() == qo).all()


def test_fp8_nan_inf_saturate(cuda_device):
    from dsl_tool_b200 import quantize_fp8
    x = torch.tensor([[1.0, float("inf"), -float("inf"), float("nan")] + [0.5] * 28], device="cuda")
    q, _ = quantize_fp8(x, "per_tensor", scale=1.0)
    b = q.cpu().numpy()[0]
    assert b[0] == 0x38 and b[1] == 0x7E and b[2] == 0xFE and (b[3] & 0x7F) == 0x7F


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_fp4_formats(cuda_device, shape, dtype, fmt):
    from dsl_tool_b200 import quantize_fp4
    xc, xo = _inputs(shape, dtype, 3)
    q, sf, gs = quantize_fp4(xc, fmt)
    if fmt == "nvfp4":
        qo, sfo, gso = O.quant_nvfp4(xo)
        assert gs.item() == gso
    else:
        qo, sfo = O.quant_mxfp4(xo)
        assert gs is None
    assert (sf.cpu().numpy() == O.swizzle_sf(sfo)).all()               # tiled layout incl. zero padding
    assert (q.cpu().numpy() == qo).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_input_that_is_only_16_byte_aligned(cuda_device, dtype):
    """The quantisers read 32 bytes per thread with one 256-bit load when every chunk sits on a 32-byte boundary and
    fall back to 16-byte loads otherwise.  A tensor that starts 16 bytes into an allocation takes the fallback: same bytes."""
    from dsl_tool_b200 import quantize_fp4, quantize_fp8
    rows, cols = 200, 512
    xc, _ = _inputs((rows, cols), dtype, 5)
    shift = 16 // xc.element_size()
    pool = torch.empty(rows * cols + shift, dtype=dtype, device="cuda")
    view = pool[shift:].view(rows, cols)
    view.copy_(xc)
    assert view.data_ptr() % 32 == 16 and xc.data_ptr() % 32 == 0
    for fmt in ("nvfp4", "mxfp4"):
        a, b = quantize_fp4(xc, fmt), quantize_fp4(view, fmt)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and (fmt == "mxfp4" or torch.equal(a[2], b[2]))
    for mode in ("per_tensor", "groupwise"):
        a, b = quantize_fp8(xc, mode), quantize_fp8(view, mode)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 32), (7, 96), (50, 768), (129, 1056), (300, 4096), (40, 8192), (9, 28672)])
def test_nvfp4_per_token_scales(cuda_device, shape, dtype):
    """global_scale="per_token": one pass; bytes, scale tiles and the per-row global scales equal the oracle's (every
    register-chunk count of both kernels - a warp per row up to 4096 bf16 elements, a CTA per row beyond and for the
    other types: rows of 32 ... 28672 elements; an all-zero row gets scale 1 and zero bytes)."""
    from dsl_tool_b200 import quantize_fp4
    xc, xo = _inputs(shape, dtype, 21)
    q, sf, gs = quantize_fp4(xc, "nvfp4", global_scale="per_token")
    pq, psf, pgs = O.quant_nvfp4(xo, "per_token")
    assert np.array_equal(gs.cpu().numpy(), pgs)
    assert np.array_equal(q.cpu().numpy(), pq)
    assert np.array_equal(O.unswizzle_sf(sf.cpu().numpy(), shape[0], shape[1] // 16), psf)
    assert np.array_equal(sf.cpu().numpy(), O.swizzle_sf(psf))          # padding bytes are zero


def test_nvfp4_per_token_ragged_groups_and_limits(cuda_device):
    from dsl_tool_b200 import quantize_fp4
    xc, xo = _inputs((300, 512), torch.bfloat16, 22)
    offs = np.array([0, 5, 5, 140, 300], np.int32)
    q, sf, gs = quantize_fp4(xc, "nvfp4", global_scale="per_token", group_offsets=torch.from_numpy(offs).cuda())
    pq, psf, pgs = O.quant_nvfp4(xo, "per_token")
    assert np.array_equal(gs.cpu().numpy(), pgs) and np.array_equal(q.cpu().numpy(), pq)
    want = O.swizzle_sf_grouped(psf, offs)
    assert np.array_equal(sf.cpu().numpy()[: want.size], want)
    for dtype, K in ((torch.bfloat16, 2048), (torch.float32, 2048), (torch.bfloat16, 8192)):    # warp per row / CTA per row
        xc, xo = _inputs((300, K), dtype, 23)
        q, sf, gs = quantize_fp4(xc, "nvfp4", global_scale="per_token", group_offsets=torch.from_numpy(offs).cuda())
        pq, psf, pgs = O.quant_nvfp4(xo, "per_token")
        assert np.array_equal(gs.cpu().numpy(), pgs) and np.array_equal(q.cpu().numpy(), pq)
        want = O.swizzle_sf_grouped(psf, offs)
        assert np.array_equal(sf.cpu().numpy()[: want.size], want)
    with pytest.raises(ValueError, match="at most"):
        quantize_fp4(torch.zeros(2, 32768 + 32, device="cuda"), "nvfp4", global_scale="per_token")
    with pytest.raises(ValueError, match="per_token"):
        quantize_fp4(xc, "mxfp4", global_scale="per_token")


def test_nvfp4_given_global_scale_and_zero_tensor(cuda_device):
    from dsl_tool_b200 import quantize_fp4
    xc, xo = _inputs((64, 128), torch.bfloat16, 4)
    q, sf, gs = quantize_fp4(xc, "nvfp4", global_scale=0.004)
    qo, sfo, _ = O.quant_nvfp4(xo, global_scale=np.float32(0.004))
    assert (q.cpu().numpy() == qo).all() and (sf.cpu().numpy() == O.swizzle_sf(sfo)).all()
    z = torch.zeros(8, 64, device="cuda")
    q, sf, gs = quantize_fp4(z, "nvfp4")
    assert gs.item() == 1.0 and not q.any() and not sf.any()
    q, sf, _ = quantize_fp4(z, "mxfp4")
    assert not q.any() and not sf.any()


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
def test_fp4_ragged_groups(cuda_device, fmt):
    from dsl_tool_b200 import quantize_fp4
    offs = np.array([0, 5, 5, 140, 300, 300], np.int32)
    xc, xo = _inputs((300, 192), torch.bfloat16, 5)
    q, sf, gs = quantize_fp4(xc, fmt, group_offsets=torch.from_numpy(offs).cuda())
    qo, sfo = (O.quant_nvfp4(xo)[:2] if fmt == "nvfp4" else O.quant_mxfp4(xo))
    want = O.swizzle_sf_grouped(sfo, offs)
    got = sf.cpu().numpy()
    assert (q.cpu().numpy() == qo).all()
    assert (got[: want.size] == want).all() and not got[want.size:].any()


def test_weight_distribution_and_determinism(cuda_device):
    from dsl_tool_b200 import quantize_fp4, quantize_fp8
    w = weights(np.random.default_rng(6), 512, 1024)
    wc = torch.from_numpy(w).cuda()
    q1, sf1, gs1 = quantize_fp4(wc, "nvfp4")
    for _ in range(2):
        q2, sf2, gs2 = quantize_fp4(wc, "nvfp4")
        assert torch.equal(q1, q2) and torch.equal(sf1, sf2) and torch.equal(gs1, gs2)
    qo, sfo, gso = O.quant_nvfp4(w)
    assert (q1.cpu().numpy() == qo).all() and gs1.item() == gso
    q, s = quantize_fp8(wc, "block128")
    qo, so = O.quant_fp8_block(w)
    assert (q.cpu().numpy() == qo).all() and (s.cpu().numpy() == so).all()


def test_transpose_bytes(cuda_device):
    from dsl_tool_b200.quantize import transpose_bytes
    b = np.random.default_rng(7).integers(0, 255, (70, 130)).astype(np.uint8)
    assert (transpose_bytes(torch.from_numpy(b).cuda()).cpu().numpy() == b.T).all()


def test_bounded_wait_reports_status_and_context_survives(cuda_device):
    from dsl_tool_b200 import _lib, quantize_fp8
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.lib().dsl_selftest_bounded_wait(st.data_ptr(), 2000, _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert st.item() == 8                               # DSL_ST_TIMEOUT_TEST
    q, s = quantize_fp8(torch.ones(4, 16, device="cuda"), "per_tensor")   # the context still works
    assert (q.cpu().numpy() == 0x7E).all()
