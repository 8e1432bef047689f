"""Outside anchors for the quantisers the reference does not define.  The reference has no NVFP4 / MXFP4 / 1x128 code
(its FP4 container is fp32 scales per 32, its FP8 quantiser per tensor), so the oracle's rules for them are this
repository's own reading of the public formats.  Where an independent implementation is installed (vLLM, flashinfer:
test-only imports), its output on the same tensor is compared.  NVFP4 against vLLM's `scaled_fp4_quant`:

  * conventions: vLLM takes the INVERSE global scale, (448 * 6) / amax, where this library stores amax / (448 * 6);
    both use one unsigned-E4M3 scale per 16 elements in the same 128 x 4 tile layout and the same nibble order;
  * arithmetic: vLLM scales with approximate reciprocals, this library with IEEE divisions, so values that sit on a
    rounding boundary of the E4M3 scale or of the e2m1 grid can land on the other side.  The test therefore asks
    for near-total agreement, not identity, and reports the fractions (a differing scale must be the neighbouring
    E4M3 code).
Skipped when vLLM or its FP4 kernel is not available on the machine."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_nvfp4_bytes_and_scale_tiles_agree_with_vllm(cuda_device):
    try:
        from vllm import _custom_ops as ops
    except Exception as exc:      # not installed, or not importable on this machine
        pytest.skip(f"vLLM is not importable: {type(exc).__name__}")
    from dsl_tool_b200 import quantize_fp4
    g = torch.Generator(device="cuda").manual_seed(5)
    M, K = 384, 1024                                  # whole 128 x 4 scale tiles: both sides fill every byte
    x = torch.randn((M, K), generator=g, device="cuda")
    x[torch.rand((M, K), generator=g, device="cuda") < 1e-3] = 20.0
    x = x.bfloat16()
    amax = x.float().abs().max()
    try:
        q_v, sf_v = ops.scaled_fp4_quant(x, (2688.0 / amax).reshape(1).float())
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"vLLM's scaled_fp4_quant does not run here: {type(exc).__name__}: {str(exc)[:120]}")
    q, sf, gs = quantize_fp4(x, "nvfp4")
    assert gs.item() == (amax / 2688.0).item()
    q_v = q_v.view(torch.uint8).reshape(M, K // 2)
    sf_v = sf_v.view(torch.uint8).reshape(-1)
    assert sf_v.numel() == sf.numel()
    same_sf = (sf_v == sf).float().mean().item()
    same_q = (q_v == q).float().mean().item()
    step = (sf_v.to(torch.int16) - sf.to(torch.int16)).abs().max().item()
    print(f"scale bytes equal: {same_sf:.6f} (largest difference {step} code), packed bytes equal: {same_q:.6f}")
    # measured on a B200: 99.30 % of the scale bytes and 99.72 % of the packed bytes identical
    assert same_sf > 0.98, same_sf                    # same layout and the same rule up to reciprocal rounding ...
    assert step <= 1, step                            # ... so a scale that differs is the neighbouring E4M3 code
    assert same_q > 0.99, same_q                      # same nibble order and grid; differences only at boundaries


def test_fp8_1x128_bytes_and_scales_equal_vllm(cuda_device):
    """1 x 128 activation groups with fp32 scales: vLLM's `per_token_group_quant_fp8(..., use_ue8m0=False)` (scale = group
    amax / 448, E4M3 round-to-nearest of x / scale) and this library agree on every byte and every scale.  On this part
    vLLM defaults to power-of-two (UE8M0) scales, a different format, hence the explicit flag."""
    try:
        from vllm.model_executor.layers.quantization.utils.fp8_utils import per_token_group_quant_fp8
    except Exception as exc:
        pytest.skip(f"vLLM is not importable: {type(exc).__name__}")
    from dsl_tool_b200 import quantize_fp8
    g = torch.Generator(device="cuda").manual_seed(6)
    x = torch.randn((384, 1024), generator=g, device="cuda").bfloat16()
    try:
        q_v, s_v = per_token_group_quant_fp8(x, 128, use_ue8m0=False)
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"vLLM's per_token_group_quant_fp8 does not run here: {type(exc).__name__}: {str(exc)[:120]}")
    q, s = quantize_fp8(x, "groupwise")
    assert torch.equal(s_v.float().contiguous(), s)
    assert torch.equal(q_v.view(torch.uint8), q)


def test_mxfp4_agrees_with_flashinfer_wherever_the_exponents_do(cuda_device):
    """MXFP4 against flashinfer's `mxfp4_quantize`.  The two differ in ONE convention, the shared exponent: this
    library takes the OCP rule, floor(log2(amax)) - 2 (values above 6 * 2^e saturate), flashinfer rounds the exponent up
    so that nothing saturates.  So the scale byte is either equal or theirs is one higher; in every block where it is
    equal, all 16 packed bytes are equal too (same e2m1 rounding, same nibble order, same 128 x 4 scale-tile layout)."""
    try:
        import flashinfer
    except Exception as exc:
        pytest.skip(f"flashinfer is not importable: {type(exc).__name__}")
    from dsl_tool_b200 import quantize_fp4
    g = torch.Generator(device="cuda").manual_seed(7)
    M, K = 384, 1024
    x = torch.randn((M, K), generator=g, device="cuda").bfloat16()
    try:
        q_f, sf_f = flashinfer.mxfp4_quantize(x)
        torch.cuda.synchronize()
    except Exception as exc:      # it compiles its kernel on first use, which needs a working toolchain on the machine
        pytest.skip(f"flashinfer's mxfp4_quantize does not run here: {type(exc).__name__}: {str(exc)[:120]}")
    q, sf, _ = quantize_fp4(x, "mxfp4")
    sf_f = sf_f.view(torch.uint8).reshape(-1)
    assert sf_f.numel() == sf.numel()
    delta = sf_f.to(torch.int16) - sf.to(torch.int16)
    assert set(torch.unique(delta).tolist()) <= {0, 1}

    def rows_by_blocks(tiles):      # 512-byte tiles of 128 rows x 4 K-blocks -> [M, K/32]
        return tiles.reshape(M // 128, (K // 32) // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(M, K // 32)
    same_scale = rows_by_blocks(sf_f) == rows_by_blocks(sf)
    same_bytes = (q_f.view(torch.uint8).reshape(M, K // 32, 16) == q.reshape(M, K // 32, 16)).all(dim=2)
    print(f"blocks with the same exponent: {same_scale.float().mean().item():.4f}")
    assert same_scale.float().mean().item() > 0.5           # measured 0.71 on N(0, 1) data
    assert bool(same_bytes[same_scale].all())
