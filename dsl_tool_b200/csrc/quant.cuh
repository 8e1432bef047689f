// Host launchers of the quantise / scale-pack kernels (definitions in quant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "dslgemm.h"

namespace dsl {
cudaError_t launch_quant_fp8(const void* x, int dtype, long long rows, long long cols, int mode, float* scale_io,
                             int scale_given, uint8_t* q, uint32_t* ws, cudaStream_t st);
cudaError_t launch_quant_fp4(const void* x, int dtype, long long rows, long long cols, int format, float* gs_io,
                             int gs_given, uint8_t* q, uint8_t* sf, size_t sf_bytes, int sf_needs_clear,
                             const int* group_offsets, int num_groups, uint32_t* ws, cudaStream_t st);
cudaError_t launch_quant_nvfp4_per_token(const void* x, int dtype, long long rows, long long cols, float* gs_out, uint8_t* q,
                                         uint8_t* sf, size_t sf_bytes, int sf_needs_clear, const int* group_offsets,
                                         int num_groups, cudaStream_t st);
cudaError_t launch_transpose_u8(const uint8_t* in, uint8_t* out, int R, int C, cudaStream_t st);
}  // namespace dsl
