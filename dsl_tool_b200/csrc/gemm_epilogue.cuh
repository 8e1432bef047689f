// Epilogue helper shared by the GEMM kernels: scale 32 consecutive accumulator columns of one
// output row, optionally fold (gate, up) column pairs into silu(gate) * up, convert, and store
// (16-byte vector stores when the row is aligned).
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

#include <float.h>

#include "gemm.cuh"
#include "ptx.cuh"

namespace dsl {

// One NVFP4 block of the result: 16 consecutive output columns of one row -> 8 packed bytes + one
// scale byte in the tile layout, with the arithmetic of the NVFP4 quantiser (quant.cu):
//   sf = ue4m3_rne(min((amax/6)/gs, 448)),  q = e2m1_rne(x * (1 / (f32(sf) * gs))).
// `sf_tile` is the 128-row scale tile the row belongs to, `rin` the row's index inside it.
__device__ __forceinline__ void store_nvfp4_block(const GemmArgs& args, int row, int ocol0, const float* x, float gs,
                                                  int sf_tile, int rin) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(x[i]));
    float t = __fdiv_rn(__fdiv_rn(m, 6.0f), gs);
    t = fminf(t, 448.0f);
    const uint32_t sfb = cvt_e4m3x2(t, 0.f) & 0xFFu;
    const float d = __fmul_rn(e4m3_to_float(sfb), gs);
    const float inv = d >= FLT_MIN ? __frcp_rn(d) : 0.f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t b = cvt_e2m1x2(__fmul_rn(x[2 * i], inv), __fmul_rn(x[2 * i + 1], inv));
        w[i >> 2] |= b << (8 * (i & 3));
    }
    uint8_t* c = static_cast<uint8_t*>(args.c);
    *reinterpret_cast<uint2*>(c + static_cast<size_t>(row) * (args.ldc >> 1) + (ocol0 >> 1)) = make_uint2(w[0], w[1]);
    const int blk = ocol0 >> 4;
    args.out_sf[(static_cast<size_t>(sf_tile) * args.out_sf_katoms + (blk >> 2)) * 512 + (rin & 31) * 16 + (rin >> 5) * 4 + (blk & 3)] =
        static_cast<uint8_t>(sfb);
}

// v: 32 fp32 accumulators (bit patterns) of row `row`, columns col0..col0+31 of group `group`.
// out = (acc * s1) * s2 [* row_scale[row]] [* col_scale[group*n + col]]
// sf_tile / rin: only read when the result is quantised (args.out_sf != nullptr).
// FULL = false compiles the activation and quantisation branches out: the group-scaled FP8 kernels hold 128
// accumulators per thread and must not pay registers (measured: spills in the promotion loop) for paths they
// take rarely; they are instantiated once without and once with those branches and the launcher chooses.
template <bool FULL>
__device__ __forceinline__ void store_chunk32_t(const GemmArgs& args, int row, int col0, int group,
                                                const uint32_t (&v)[32], float s1, float s2, float rs, bool vec_ok,
                                                int sf_tile = 0, int rin = 0) {
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
    if (FULL && args.act != DSL_ACT_NONE) {
        // columns (2j, 2j+1) = (gate_j, up_j) -> output column col0/2 + j of an [m, n/2] result;
        // SwiGLU: silu(x) = x / (1 + exp(-x)) (cuda/activations/fused_gated_activations.cu:27-29).
        // GeGLU: gelu(x) = 0.5 x (1 + tanh(c (x + k x^3))) (:32-37) = x / (1 + exp(-2c (x + k x^3))), the same shape.
        const bool geglu = args.act == DSL_ACT_GEGLU;
        float o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float g = f[2 * j];
            const float z = geglu ? 1.5957691216f * (g + 0.044715f * g * g * g) : g;
            // fast exponential and division (a few ulp): the epilogue must stay shorter than a tile's MMAs
            o[j] = __fmul_rn(__fdividef(g, 1.0f + __expf(-z)), f[2 * j + 1]);
        }
        const int c0 = col0 >> 1;
        if (args.out_sf != nullptr) {     // n/2 is a multiple of 16 here, so the 16 outputs are one whole block
            if (col0 < args.n) store_nvfp4_block(args, row, c0, o, args.out_gs_dev != nullptr ? *args.out_gs_dev : args.out_gs, sf_tile, rin);
            return;
        }
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
    if (FULL && args.out_sf != nullptr) {         // n is a multiple of 16: one or two whole blocks in this chunk
        const float gs = args.out_gs_dev != nullptr ? *args.out_gs_dev : args.out_gs;
        if (col0 < args.n) store_nvfp4_block(args, row, col0, f, gs, sf_tile, rin);
        if (col0 + 16 < args.n) store_nvfp4_block(args, row, col0 + 16, f + 16, gs, sf_tile, rin);
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

__device__ __forceinline__ void store_chunk32(const GemmArgs& args, int row, int col0, int group,
                                              const uint32_t (&v)[32], float s1, float s2, float rs, bool vec_ok,
                                              int sf_tile = 0, int rin = 0) {
    store_chunk32_t<true>(args, row, col0, group, v, s1, s2, rs, vec_ok, sf_tile, rin);
}

// Plain bf16 result, stored by the whole warp: every lane scales and converts its own row's 32 columns
// (64 bytes), the 32 rows are exchanged through 2 KB of shared memory (16-byte pieces, XOR-placed so that
// neither side has bank conflicts), and every store instruction then writes 8 rows x 64 contiguous bytes
// instead of 16 bytes in each of 32 rows - a quarter of the memory transactions.  Short-K tiles, whose MMAs
// are no longer than their epilogue, are where this shows (MoE down projection).  Call with all 32 lanes;
// rows at or beyond row_end are not written.
__device__ __forceinline__ void store_chunk32_bf16_warp(const GemmArgs& args, uint8_t* scratch, int row_base, int row_end,
                                                        int col0, int group, const uint32_t (&v)[32], float s1, float s2,
                                                        float rs, int lane) {
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
        for (int i = 0; i < 32; ++i) f[i] = __fmul_rn(f[i], cs[col0 + i]);
    }
    const int swz = (lane >> 1) & 3;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[8 * p + 2 * j], f[8 * p + 2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(scratch + lane * 64 + 16 * (p ^ swz)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncwarp();
    const int p = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rr = (lane >> 2) + 8 * i;
        const uint4 d = *reinterpret_cast<const uint4*>(scratch + rr * 64 + 16 * (p ^ ((rr >> 1) & 3)));
        const int row = row_base + rr;
        if (row < row_end)
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.c) + static_cast<size_t>(row) * args.ldc + col0 + 8 * p) = d;
    }
    __syncwarp();
}

}  // namespace dsl
