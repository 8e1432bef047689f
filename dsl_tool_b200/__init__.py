"""B200 (sm_100a) quantised-GEMM backend: `gemm.fp8_gemm`, `gemm.fp4_gemm`, `gemm.grouped_gemm`.

Python host code over a C-ABI CUDA library (libdslgemm.so, built in-tree by
`python -m dsl_tool_b200.build`).  The operators raise when the library or a CUDA device is
missing; there is no CPU path.
"""
from .gemm_kernels import bf16_gemm, fp4_gemm, fp8_gemm, grouped_gemm, linear
from .quantize import PackedWeight, pack_weight, quantize_fp4, quantize_fp4_ref32, quantize_fp8
from .moe import MoEWeights, moe_forward
from .host_io import HostPipeline
from .weight_store import WeightCache, cached_pack, load_packed, save_packed

__all__ = ["fp8_gemm", "fp4_gemm", "grouped_gemm", "bf16_gemm", "linear", "PackedWeight", "pack_weight",
           "quantize_fp8", "quantize_fp4", "quantize_fp4_ref32", "WeightCache", "cached_pack", "load_packed", "save_packed", "MoEWeights", "moe_forward", "HostPipeline"]
