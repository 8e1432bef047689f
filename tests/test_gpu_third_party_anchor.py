"""An outside anchor for the NVFP4 quantiser.  The reference has no NVFP4 code (its FP4 container is fp32 scales per
32), so the oracle's NVFP4 rule is this repository's own reading of the public format.  Where an independent
implementation is installed (vLLM's `scaled_fp4_quant`, test-only import), its output on the same tensor is compared:

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
