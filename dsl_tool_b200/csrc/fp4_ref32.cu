// The reference's own FP4 container ("NVFP4"/"MXFP4" of cuda/gemm/fp4_gemm.cu are one format): e2m1
// nibbles with an fp32 scale per 32 contiguous elements.  fp32 scales per 32 elements cannot ride in
// the block-scaled tensor-core instruction, so this drop-in path runs on the integer dot-product
// units instead: doubled e2m1 values are small integers, the 32-element group sum is an exact
// dp4a sum, and each group is then folded in as acc = fma(ga * sa, sb, acc) in ascending group
// order - the same rounding sequence as fp4_gemm_kernel (fp4_gemm.cu:95-137), so results are
// bit-identical to the reference kernel's.
//
//   quantize_fp32_to_nvfp4 (fp4_gemm.cu:50-90): scale = max(amax/6, 1e-12), v = x * (1/scale),
//   nearest table entry, ties to the LOWER index (toward zero), -0 never produced.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "dslgemm.h"
#include "ptx.cuh"

namespace dsl {

template <typename T> __device__ __forceinline__ float ld_f32(const T* p);
template <> __device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ld_f32<__half>(const __half* p) { return __half2float(*p); }

// Nearest e2m1 code with the reference's tie rule (first minimum of a linear scan, fp4_gemm.cu:80-87).
__device__ __forceinline__ uint32_t e2m1_ref_lut(float v) {
    const float a = fabsf(v);
    const uint32_t code = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    return (code != 0u && v < 0.f) ? code + 8u : code;
}

// One thread per 32-element block, as the reference kernel; the flat buffer may end in a short block.
template <typename T>
__global__ void __launch_bounds__(256)
quant_fp4_ref32_kernel(const T* __restrict__ x, long long n, uint8_t* __restrict__ q, float* __restrict__ scales) {
    const long long b = blockIdx.x * 256ll + threadIdx.x;
    const long long start = b * 32;
    if (start >= n) return;
    const int len = static_cast<int>(n - start < 32 ? n - start : 32);
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = i < len ? ld_f32<T>(x + start + i) : 0.f;
        amax = fmaxf(amax, fabsf(v[i]));
    }
    float scale = __fdiv_rn(amax, 6.0f);
    if (scale < 1e-12f) scale = 1e-12f;
    scales[b] = scale;
    const float inv = __fdiv_rn(1.0f, scale);
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        if (i < len) {
            const uint32_t q0 = e2m1_ref_lut(__fmul_rn(v[i], inv));
            const uint32_t q1 = e2m1_ref_lut(i + 1 < len ? __fmul_rn(v[i + 1], inv) : 0.f);
            q[(start + i) / 2] = static_cast<uint8_t>((q1 << 4) | q0);
        }
    }
}

// doubled e2m1 magnitudes {0,1,2,3,4,6,8,12}; sign from bit 3
__device__ __forceinline__ int nib_x2(uint32_t nib) {
    const int mag = (0x0C08060403020100ull >> ((nib & 7u) * 8)) & 0xFF;
    return (nib & 8u) ? -mag : mag;
}

// C[M,N] fp32; A packed [M, K/2] (pairs along K); B packed [K, N/2] (pairs along N);
// sa [M, K/32], sb [K/32, N].  64 x 64 output tile per CTA, 4 x 4 outputs per thread.
__global__ void __launch_bounds__(256)
gemm_fp4_ref32_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B, float* __restrict__ C,
                      const float* __restrict__ sa, const float* __restrict__ sb, int M, int N, int K) {
    __shared__ int As[64][9];    // [row][8 words of 4 doubled values along k] (+1 pad)
    __shared__ int Bs[64][9];    // [col][8 words along k]
    __shared__ float sSa[64], sSb[64];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int ng = K / 32;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    int8_t* Bs8 = reinterpret_cast<int8_t*>(&Bs[0][0]);
    for (int g = 0; g < ng; ++g) {
        __syncthreads();
        {   // A: 64 rows x 16 bytes; thread t -> row t/4, 4 bytes (8 values = 2 words)
            const int r = threadIdx.x >> 2, part = threadIdx.x & 3;
            uint32_t w = 0;
            if (m0 + r < M) w = *reinterpret_cast<const uint32_t*>(A + (static_cast<size_t>(m0 + r) * K + g * 32) / 2 + part * 4);
            int lo = 0, hi = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                lo |= (nib_x2((w >> (4 * e)) & 0xF) & 0xFF) << (8 * e);
                hi |= (nib_x2((w >> (16 + 4 * e)) & 0xF) & 0xFF) << (8 * e);
            }
            As[r][part * 2] = lo;
            As[r][part * 2 + 1] = hi;
        }
        {   // B: 32 k-rows x 32 bytes (64 columns); thread t -> k = t/8, 4 bytes = 8 columns
            const int k = threadIdx.x >> 3, part = threadIdx.x & 7;
            const int c0 = part * 8;
            uint32_t w = 0;
            if (n0 + c0 < N) w = *reinterpret_cast<const uint32_t*>(B + (static_cast<size_t>(g * 32 + k) * N + n0 + c0) / 2);
#pragma unroll
            for (int e = 0; e < 8; ++e) Bs8[(c0 + e) * 36 + k] = static_cast<int8_t>(nib_x2((w >> (4 * e)) & 0xF));
        }
        if (threadIdx.x < 64) sSa[threadIdx.x] = (m0 + threadIdx.x < M) ? sa[static_cast<size_t>(m0 + threadIdx.x) * ng + g] : 0.f;
        else if (threadIdx.x < 128) {
            const int c = threadIdx.x - 64;
            sSb[c] = (n0 + c < N) ? sb[static_cast<size_t>(g) * N + n0 + c] : 0.f;
        }
        __syncthreads();
        int isum[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) isum[i][j] = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            int a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[ty * 4 + i][w];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[tx * 4 + j][w];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) isum[i][j] = __dp4a(a[i], b[j], isum[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float sai = sSa[ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float ga = static_cast<float>(isum[i][j]) * 0.25f;          // exact group sum
                acc[i][j] = fmaf(__fmul_rn(ga, sai), sSb[tx * 4 + j], acc[i][j]);   // fp4_gemm.cu:133
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = m0 + ty * 4 + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < N) C[static_cast<size_t>(r) * N + c] = acc[i][j];
        }
    }
}

}  // namespace dsl

using namespace dsl;

extern "C" int dsl_quant_fp4_ref32(const void* x, int dtype, long long n, uint8_t* q_out, float* scales_out, void* stream) {
    if (x == nullptr || q_out == nullptr || scales_out == nullptr) return DSL_ERR_NULL;
    if (dtype < DSL_F32 || dtype > DSL_F16) return DSL_ERR_ENUM;
    if (n < 0 || n > (1ll << 40)) return DSL_ERR_SHAPE;
    if (n == 0) return 0;
    const long long blocks = (n + 31) / 32;
    const unsigned grid = static_cast<unsigned>((blocks + 255) / 256);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == DSL_F32) quant_fp4_ref32_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), n, q_out, scales_out);
    else if (dtype == DSL_BF16) quant_fp4_ref32_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, q_out, scales_out);
    else quant_fp4_ref32_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), n, q_out, scales_out);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int dsl_gemm_fp4_ref32(const uint8_t* A, const uint8_t* B, float* C, const float* scale_a, const float* scale_b,
                                  int M, int N, int K, void* stream) {
    if (A == nullptr || B == nullptr || C == nullptr || scale_a == nullptr || scale_b == nullptr) return DSL_ERR_NULL;
    if (M < 0 || N < 0 || K <= 0 || K % 32 != 0 || N % 8 != 0) return DSL_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) & 3u) || (reinterpret_cast<uintptr_t>(B) & 3u)) return DSL_ERR_ALIGN;
    if (M == 0 || N == 0) return 0;
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    gemm_fp4_ref32_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(A, B, C, scale_a, scale_b, M, N, K);
    return static_cast<int>(cudaGetLastError());
}
