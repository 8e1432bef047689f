"""`KernelDispatcher.run_from_spec` with backend "cuda" for the three kernel names.  GPU."""
import base64

import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests.helpers import REL_FROB_TOL, activations, rel_frobenius, weights

pytestmark = pytest.mark.gpu


def _spec(a: np.ndarray, dtype: str):
    return {"shape": list(a.shape), "dtype": dtype, "data": base64.b64encode(np.ascontiguousarray(a).tobytes()).decode()}


def test_run_from_spec_fp8_config0(cuda_device):
    """The per-tensor plumbing configuration: fp32 N(0,1) A and B, per-tensor scale amax/448, M=N=K=1024."""
    from dsl_tool_b200.dispatcher import KernelDispatcher
    rng = np.random.default_rng(0)
    a = rng.standard_normal((1024, 1024)).astype(np.float32)
    b = rng.standard_normal((1024, 1024)).astype(np.float32)       # [K, N]
    d = KernelDispatcher()
    res = d.run_from_spec("gemm.fp8_gemm", "cuda", [_spec(a, "float32"), _spec(b, "float32")], {"out_dtype": "bfloat16"})
    assert res.backend == "cuda" and res.kernel_name == "gemm.fp8_gemm" and "B200" in res.device_info
    out = res.to_dict()["output"]
    assert out["dtype"] == "bfloat16" and out["shape"] == [1024, 1024]
    got = np.frombuffer(base64.b64decode(out["data"]), np.float32).reshape(1024, 1024)
    qa, sa = O.quant_fp8_per_tensor(a)
    qb, sb = O.quant_fp8_per_tensor(np.ascontiguousarray(b.T))
    want = O.bf16_round(O.gemm_fp8_per_tensor(qa, qb, sa, sb))
    assert rel_frobenius(got, want) <= 4e-3
    res32 = d.run_from_spec("gemm.fp8_gemm", "cuda", [_spec(a, "float32"), _spec(b, "float32")], {})
    assert res32.output.dtype == torch.float32
    assert rel_frobenius(res32.output.cpu().numpy(), O.gemm_fp8_per_tensor(qa, qb, sa, sb)) <= REL_FROB_TOL


def test_run_from_spec_fp4_and_grouped(cuda_device):
    from dsl_tool_b200.dispatcher import KernelDispatcher
    rng = np.random.default_rng(1)
    a = activations(rng, 64, 256)
    b = np.ascontiguousarray(weights(rng, 128, 256).T)             # [K, N]
    d = KernelDispatcher()
    res = d.run_from_spec("gemm.fp4_gemm", "cuda", [_spec(a, "float32"), _spec(b, "float32")], {"use_mxfp4": True})
    want = O.gemm_mxfp4(*O.quant_mxfp4(a), *O.quant_mxfp4(np.ascontiguousarray(b.T)))
    assert rel_frobenius(res.output.cpu().numpy(), want) <= REL_FROB_TOL
    ga = rng.standard_normal((4, 32, 64)).astype(np.float32)
    gb = rng.standard_normal((4, 64, 48)).astype(np.float32)
    res = d.run_from_spec("gemm.grouped_gemm", "cuda", [_spec(ga, "bfloat16"), _spec(gb, "bfloat16")], {"num_groups": 4})
    assert res.output.shape == (4, 32, 48) and res.output.dtype == torch.bfloat16
    ab = O.bf16_round(ga)
    bb = O.bf16_round(gb)
    assert rel_frobenius(res.output.float().cpu().numpy(), O.bf16_round(np.einsum("gmk,gkn->gmn", ab, bb))) <= 4e-3


def test_kernel_errors_are_wrapped(cuda_device):
    from dsl_tool_b200.dispatcher import KernelDispatcher
    with pytest.raises(RuntimeError, match=r"Kernel 'gemm.fp8_gemm' \[cuda\] raised: inner dimensions"):
        KernelDispatcher().run_from_spec("gemm.fp8_gemm", "cuda", [{"shape": [8, 64], "dtype": "float32", "fill": "ones"},
                                                                    {"shape": [32, 8], "dtype": "float32", "fill": "ones"}], {})
