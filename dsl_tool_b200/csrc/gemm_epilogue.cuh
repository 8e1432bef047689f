// Epilogue helper shared by the GEMM kernels: scale 32 consecutive accumulator columns of one
// output row, optionally fold (gate, up) column pairs into silu(gate) * up, convert, and store
// (16-byte vector stores when the row is aligned).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include "gemm.cuh"

namespace dsl {

// v: 32 fp32 accumulators (bit patterns) of row `row`, columns col0..col0+31 of group `group`.
// out = (acc * s1) * s2 [* row_scale[row]] [* col_scale[group*n + col]]
__device__ __forceinline__ void store_chunk32(const GemmArgs& args, int row, int col0, int group,
                                              const uint32_t (&v)[32], float s1, float s2, float rs, bool vec_ok) {
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float x = __fmul_rn(__fmul_rn(__uint_as_float(v[i]), s1), s2);
        if (args.row_scale != nullptr) x = __fmul_rn(x, rs);
        f[i] = x;
    }
    if (args.col_scale != nullptr) {
        const float* cs = args.col_scale + static_cast<size_t>(group) * args.n;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (col0 + i < args.n) f[i] = __fmul_rn(f[i], cs[col0 + i]);
    }
    if (args.act == DSL_ACT_SWIGLU) {
        // columns (2j, 2j+1) = (gate_j, up_j) -> output column col0/2 + j of an [m, n/2] result;
        // silu(x) = x / (1 + exp(-x)) as cuda/activations/fused_gated_activations.cu:27-29, in fp32
        float o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float g = f[2 * j];
            // fast exponential and division (a few ulp): the epilogue must stay shorter than a tile's MMAs
            o[j] = __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), f[2 * j + 1]);
        }
        const int c0 = col0 >> 1;
        const size_t off = static_cast<size_t>(row) * args.ldc + c0;
        if (vec_ok && col0 + 32 <= args.n) {
            if (args.out_bf16) {
                uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.c) + off);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 p = __floats2bfloat162_rn(o[8 * i + 2 * j], o[8 * i + 2 * j + 1]);
                        w[j] = *reinterpret_cast<uint32_t*>(&p);
                    }
                    dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
                float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.c) + off);
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (col0 + 2 * j + 1 < args.n) {
                    if (args.out_bf16) static_cast<__nv_bfloat16*>(args.c)[off + j] = __float2bfloat16_rn(o[j]);
                    else static_cast<float*>(args.c)[off + j] = o[j];
                }
            }
        }
        return;
    }
    const size_t off = static_cast<size_t>(row) * args.ldc + col0;
    if (vec_ok && col0 + 32 <= args.n) {
        if (args.out_bf16) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.c) + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 p = __floats2bfloat162_rn(f[8 * i + 2 * j], f[8 * i + 2 * j + 1]);
                    w[j] = *reinterpret_cast<uint32_t*>(&p);
                }
                dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        } else {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.c) + off);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (col0 + i < args.n) {
                if (args.out_bf16) static_cast<__nv_bfloat16*>(args.c)[off + i] = __float2bfloat16_rn(f[i]);
                else static_cast<float*>(args.c)[off + i] = f[i];
            }
        }
    }
}

}  // namespace dsl
