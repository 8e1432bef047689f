"""NVFP4 quantisation of the GEMM result inside the epilogue (optionally after the fused SwiGLU): the
packed bytes and scale tiles must be exactly what the stand-alone quantiser makes of the fp32 result
with the same global scale, so the next FP4 GEMM can take them as its A operand unchanged."""
import numpy as np
import pytest
import torch

import dsl_tool_b200 as D
from dsl_tool_b200 import _lib
from dsl_tool_b200.gemm_kernels import gemm_fp4_quantized
from oracle import quant_oracle as O
from tests.helpers import activations, moe_offsets, weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4", "fp8", "bf16"])
@pytest.mark.parametrize("M", [40, 300])                      # 1-CTA kernel / CTA-pair kernel
@pytest.mark.parametrize("act", [None, "swiglu"])
def test_quantised_result_equals_quantiser(cuda_device, fmt, M, act):
    rng = np.random.default_rng(M + (7 if act else 0))
    N, K = 384, 512
    a = torch.from_numpy(activations(rng, M, K, outliers=True)).bfloat16().to(cuda_device)
    w = torch.from_numpy(weights(rng, N, K, std=0.05)).bfloat16().to(cuda_device)
    pw = D.pack_weight(w, fmt, gate_up_interleave=act is not None)
    ref = D.linear(a, pw, activation=act)                     # fp32 result of the same kernel path
    gs = ref.abs().amax() / 2688.0
    p, sf, g = D.linear(a, pw, activation=act, out_dtype="nvfp4", out_global_scale=gs)
    _lib.check_status()
    pe, sfe, ge = D.quantize_fp4(ref, "nvfp4", global_scale=gs)
    assert p.dtype == torch.uint8 and tuple(p.shape) == (M, ref.shape[1] // 2)
    assert torch.equal(p, pe) and torch.equal(sf, sfe) and torch.equal(g, ge)
    if M == 40 and fmt == "nvfp4":                            # and the oracle agrees with both
        po, sfo, _ = O.quant_nvfp4(ref.cpu().numpy(), global_scale=np.float32(gs.item()))
        assert np.array_equal(p.cpu().numpy(), po)
        assert np.array_equal(sf.cpu().numpy(), O.swizzle_sf(sfo).reshape(-1))


def test_two_layer_moe_chain(cuda_device):
    """gate/up projection with SwiGLU and NVFP4 output feeding the down projection, ragged experts: equal to
    the same chain with the activation tensor written out in fp32 and quantised by the stand-alone kernel."""
    rng = np.random.default_rng(31)
    G, K, H, D2 = 5, 256, 128, 192
    offs_np = moe_offsets(rng, 80, G, 4, bias_std=1.0)
    offs_np[2] = offs_np[1]                                   # an empty expert
    offs = torch.from_numpy(offs_np).to(cuda_device)
    M = int(offs_np[-1])
    a = torch.from_numpy(activations(rng, M, K)).bfloat16().to(cuda_device)
    w1 = torch.from_numpy((rng.standard_normal((G, 2 * H, K)) * 0.05).astype(np.float32)).bfloat16().to(cuda_device)
    w2 = torch.from_numpy((rng.standard_normal((G, D2, H)) * 0.05).astype(np.float32)).bfloat16().to(cuda_device)
    p1 = D.pack_weight(w1, "nvfp4", gate_up_interleave=True)
    p2 = D.pack_weight(w2, "nvfp4")
    h32 = D.linear(a, p1, expert_offsets=offs, activation="swiglu")
    gs = h32.abs().amax() / 2688.0
    hp, hsf, hg = D.linear(a, p1, expert_offsets=offs, activation="swiglu", out_dtype="nvfp4", out_global_scale=gs)
    ep, esf, eg = D.quantize_fp4(h32, "nvfp4", global_scale=gs, group_offsets=offs)
    assert torch.equal(hp, ep) and torch.equal(hsf, esf)
    down = lambda p, sf, g: gemm_fp4_quantized(p, p2.q, sf, p2.scale, format="nvfp4", n=D2, global_scale_a=g,
                                               global_scale_b=p2.global_scale, expert_offsets=offs)
    assert torch.equal(down(hp, hsf, hg), down(ep, esf, eg))
    _lib.check_status()


def test_argument_checks(cuda_device):
    a = torch.randn(8, 256, device=cuda_device)
    w = torch.randn(136, 256, device=cuda_device)              # 136 columns: not a multiple of 16
    with pytest.raises(ValueError):
        D.linear(a, D.pack_weight(w, "fp8"), out_dtype="nvfp4", out_global_scale=1.0)
    w = torch.randn(128, 256, device=cuda_device)
    with pytest.raises(ValueError):
        D.linear(a, D.pack_weight(w, "fp8"), out_dtype="nvfp4")                       # no global scale
    with pytest.raises(ValueError):
        D.linear(a, D.pack_weight(w, "fp8_block128"), out_dtype="nvfp4", out_global_scale=1.0)
