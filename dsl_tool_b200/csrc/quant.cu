// Activation / weight quantise + scale-pack kernels (HBM-bound; one vectorised pass over
// the input, 16 elements per thread, packed 8/16-byte stores).
//
// Arithmetic is IEEE fp32 throughout (explicit __fdiv_rn / __frcp_rn / __fmul_rn, never
// fast-math) so that the bytes are identical to the CPU oracle's:
//   FP8  : scale = max(amax/448, 1e-12), q = e4m3_rn_satfinite(x / scale)
//          (rule of the reference quantiser, cuda/gemm/fp8_gemm.cu:119-144), applied per
//          tensor, per 1x128 K-group, or per 128x128 block.
//   NVFP4: gs = amax_tensor/2688 (1 if zero); sf = ue4m3(min((amax16/6)/gs, 448));
//          inv = 1/(f32(sf)*gs) (0 if that product is below FLT_MIN); q = e2m1_rn(x*inv).
//   MXFP4: e = clamp(exponent(amax32) - 2, -127, 127); byte = e+127; q = e2m1_rn(x * 2^-e).
// FP4 nibble order follows cuda/gemm/fp4_gemm.cu:46,88: low nibble = even element.
// Scale bytes are written straight into the 512-byte (128 rows x 4 K-blocks) tile layout the
// block-scaled MMA consumes: byte (r, c) of a tile at (r%32)*16 + (r/32)*4 + c.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>

#include "gemm_tiles.cuh"
#include "ptx.cuh"
#include "quant.cuh"

namespace dsl {

// ---- 16-element vector loads ------------------------------------------------------------
template <typename T> struct dsl_is_half { static constexpr bool value = false; };
template <> struct dsl_is_half<__half> { static constexpr bool value = true; };
template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 t = __ldg(q + i);
        v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 t = __ldg(q + i);
        uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
}
template <>
__device__ __forceinline__ void load16<__half>(const __half* p, float (&v)[16]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint4 t = __ldg(q + i);
        uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[j]));
            v[8 * i + 2 * j] = f.x;
            v[8 * i + 2 * j + 1] = f.y;
        }
    }
}
// The same 16 elements with 256-bit loads (one for 16-bit types, two for fp32): a warp's request then covers whole
// 128-byte lines instead of every other 16 bytes of them, which halves the requests the L1 has to replay for these
// streaming kernels.  The address must be 32-byte aligned (`wide` is decided on the host from the base pointer and the
// row pitch); the data is read once, so it bypasses L1 allocation.
__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}
template <typename T>
__device__ __forceinline__ void load16w(const T* p, float (&v)[16], bool wide) {
    if (!wide) { load16<T>(p, v); return; }
    if (sizeof(T) == 4) {
        uint32_t a[8], b[8];
        ldg256(p, a);
        ldg256(reinterpret_cast<const uint8_t*>(p) + 32, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) { v[i] = __uint_as_float(a[i]); v[8 + i] = __uint_as_float(b[i]); }
    } else {
        uint32_t w[8];
        ldg256(p, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (sizeof(T) == 2 && !dsl_is_half<T>::value) {
                v[2 * j] = __uint_as_float(w[j] << 16);
                v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            } else {
                float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[j]));
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
        }
    }
}
// ---- one thread's 16 elements --------------------------------------------------------------
// Generic form: 16 floats.  bf16 (the activations' usual type) has a form that keeps the raw 8 words: the block
// maximum comes from packed |x| / max on bf16 pairs (exact: they are comparisons), and the e2m1 conversion widens,
// scales two values per instruction (mul.rn.f32x2, the same bits as two __fmul_rn) and merges the nibble pairs with
// byte permutes.  These kernels run at 0.76 instructions per scheduler and cycle (ncu), so instructions are time.
__device__ __forceinline__ void mul2(float a0, float a1, unsigned long long s2, float& r0, float& r1) {
    unsigned long long a, r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(s2));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r0), "=f"(r1) : "l"(r));
}
__device__ __forceinline__ uint32_t pack4(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
    return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}
template <typename T>
struct Chunk16 {
    float v[16];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    __device__ __forceinline__ void load(const T* p, bool wide) { load16w<T>(p, v, wide); }
    __device__ __forceinline__ float amax() const {
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
        return m;
    }
    __device__ __forceinline__ uint2 quant_e2m1(float inv) const {
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t b = cvt_e2m1x2(__fmul_rn(v[2 * i], inv), __fmul_rn(v[2 * i + 1], inv));
            w[i >> 2] |= b << (8 * (i & 3));
        }
        return make_uint2(w[0], w[1]);
    }
    __device__ __forceinline__ void to_float(float (&o)[16]) const {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = v[i];
    }
};
template <>
struct Chunk16<__nv_bfloat16> {
    uint32_t w[8];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = 0u;
    }
    __device__ __forceinline__ void load(const __nv_bfloat16* p, bool wide) {
        if (wide) {
            ldg256(p, w);
        } else {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(p)), b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
    }
    // max(|a|, |b|) per half with the signs xor-ed into the result: the magnitude is what the next step looks at, so
    // the eight words chain without masking the signs first (a NaN half yields the other operand, as fmaxf does)
    static __device__ __forceinline__ uint32_t absmax2(uint32_t a, uint32_t b) {
        uint32_t d;
        asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
        return d;
    }
    __device__ __forceinline__ float amax() const {
        const uint32_t m = absmax2(absmax2(absmax2(w[0], w[1]), absmax2(w[2], w[3])),
                                   absmax2(absmax2(w[4], w[5]), absmax2(w[6], w[7]))) & 0x7FFF7FFFu;
        return fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xFFFF0000u));
    }
    __device__ __forceinline__ uint2 quant_e2m1(float inv) const {
        unsigned long long s2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "f"(inv));
        uint32_t b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float lo, hi;
            mul2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u), s2, lo, hi);
            b[i] = cvt_e2m1x2(lo, hi);
        }
        return make_uint2(pack4(b[0], b[1], b[2], b[3]), pack4(b[4], b[5], b[6], b[7]));
    }
    __device__ __forceinline__ void to_float(float (&o)[16]) const {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

__device__ __forceinline__ float amax16(const float (&v)[16]) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
}
// max(amax / 448, 1e-12).  The division is RN(amax * RN(1/448)) plus one residual correction, which equals the IEEE
// quotient for every amax from 2^-100 up (checked exhaustively on the CPU: oracle/quotient_check.c, mode 4); below that
// both are far under 1e-12, and an infinite amax (its residual would be NaN) keeps the infinite first product.
__device__ __forceinline__ float fp8_scale_from_amax(float amax) {
    constexpr float r448 = 0x1.24924ap-9f;                                   // RN(1/448)
    const float q0 = __fmul_rn(amax, r448);
    float s = __fmaf_rn(__fmaf_rn(-q0, 448.0f, amax), r448, q0);
    s = q0 > 3.0e38f ? q0 : s;
    return s < 1e-12f ? 1e-12f : s;
}
// x / s for the E4M3 conversion without a division per element.  With y = RN(1/s) shared by the
// 16 elements, q0 = RN(x*y) is within 2 ulp of the quotient; one residual correction
// (r = x - q*s exactly, by FMA; q' = RN(q + r*y)) brings it within half an ulp plus a sliver, and a
// second one gives the correctly rounded quotient (Markstein's theorem: a faithful q and a correctly
// rounded reciprocal suffice), i.e. the very value __fdiv_rn returns.  The residual is exact unless
// it underflows, which needs |x| < 2^-125; with a scale of at least 1e-12 such a quotient is below
// 2^-85, far under the smallest E4M3 rounding boundary (2^-10), and converts to zero either way.
// Scales the library derives are never smaller; a caller-given scale can be (its reciprocal may even
// overflow), so quant16_e4m3 takes this path only for scales inside [1e-12, 3e38] and divides for
// real otherwise.
// Two values of q0 need care: a zero (the zero residual is +0 and would turn -0 into +0) and an infinity (Inf - Inf
// poisons the residual).  With a scale DERIVED from the maximum of the very elements being divided, |x / s| <= 448 and
// x is never infinite next to a finite scale, so only the zero remains, and since s > 0 the quotient simply takes the
// sign of x (one logic instruction per element; GIVEN = false).  With a scale the caller GIVES, x * y can overflow,
// and both are caught as the fixed points of q -> 2q (GIVEN = true).  A NaN stays a NaN through the corrections.
// Written for two elements at a time with the packed fp32 instructions (mul / fma / add .f32x2: each half is the
// IEEE operation of the scalar form q0 = x*y, q1 = fma(fma(-q0, s, x), y, q0), q2 likewise from q1, and
// fma(-q, s, x) == fma(q, -s, x) bit for bit), which halves the instruction count of the E4M3 quantisers - they run
// close to the issue limit.
template <bool GIVEN>
__device__ __forceinline__ void div2_for_e4m3(float x0, float x1, unsigned long long neg_s2, unsigned long long inv2, float& r0,
                                              float& r1) {
    unsigned long long x, q0, q1, q2, r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q0) : "l"(x), "l"(inv2));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(q0), "l"(neg_s2), "l"(x));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q1) : "l"(r), "l"(inv2), "l"(q0));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(q1), "l"(neg_s2), "l"(x));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q2) : "l"(r), "l"(inv2), "l"(q1));
    float b0, b1;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(b0), "=f"(b1) : "l"(q2));
    if (GIVEN) {
        unsigned long long d;
        asm("add.rn.f32x2 %0, %1, %1;" : "=l"(d) : "l"(q0));
        float a0, a1, d0, d1;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(q0));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
        r0 = d0 == a0 ? a0 : b0;
        r1 = d1 == a1 ? a1 : b1;
    } else {
        r0 = __uint_as_float((__float_as_uint(b0) & 0x7FFFFFFFu) | (__float_as_uint(x0) & 0x80000000u));
        r1 = __uint_as_float((__float_as_uint(b1) & 0x7FFFFFFFu) | (__float_as_uint(x1) & 0x80000000u));
    }
}
template <bool GIVEN>
__device__ __forceinline__ uint4 quant16_e4m3(const float (&v)[16], float s) {
    uint32_t w[4];
    if (s >= 1e-12f && s <= 3.0e38f) {
        const float inv = __frcp_rn(s);
        const float ns = -s;
        unsigned long long inv2, neg_s2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(inv2) : "f"(inv));
        asm("mov.b64 %0, {%1, %1};" : "=l"(neg_s2) : "f"(ns));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float a, b, c, d;
            div2_for_e4m3<GIVEN>(v[4 * i], v[4 * i + 1], neg_s2, inv2, a, b);
            div2_for_e4m3<GIVEN>(v[4 * i + 2], v[4 * i + 3], neg_s2, inv2, c, d);
            w[i] = __byte_perm(cvt_e4m3x2(a, b), cvt_e4m3x2(c, d), 0x5410);
        }
    } else {   // an infinite scale (an Inf among the inputs: 0 * Inf would poison the residual), or a given
               // scale too small for the residual argument above (also zero, negative, NaN): divide for real
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t lo = cvt_e4m3x2(__fdiv_rn(v[4 * i], s), __fdiv_rn(v[4 * i + 1], s));
            uint32_t hi = cvt_e4m3x2(__fdiv_rn(v[4 * i + 2], s), __fdiv_rn(v[4 * i + 3], s));
            w[i] = lo | (hi << 16);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ uint2 quant16_e2m1(const float (&v)[16], float inv) {
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t b = cvt_e2m1x2(__fmul_rn(v[2 * i], inv), __fmul_rn(v[2 * i + 1], inv));
        w[i >> 2] |= b << (8 * (i & 3));
    }
    return make_uint2(w[0], w[1]);
}

// ---- tensor amax -------------------------------------------------------------------------
// Non-negative floats order like their bit patterns, so the reduction is an integer
// atomicMax (same trick as cuda/gemm/fp8_gemm.cu:132) and the result is order-independent.
template <typename T>
__global__ void __launch_bounds__(256) amax_kernel(const T* __restrict__ x, size_t n, uint32_t* amax_bits, bool wide) {
    float m = 0.f;
    const size_t nvec = n / 16;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {    // four chunks (128 bytes of bf16) in flight per thread
        Chunk16<T> a, b, c, d;
        a.load(x + i * 16, wide);
        b.load(x + (i + stride) * 16, wide);
        c.load(x + (i + 2 * stride) * 16, wide);
        d.load(x + (i + 3 * stride) * 16, wide);
        m = fmaxf(fmaxf(m, fmaxf(a.amax(), b.amax())), fmaxf(c.amax(), d.amax()));
    }
    for (; i < nvec; i += stride) {
        Chunk16<T> a;
        a.load(x + i * 16, wide);
        m = fmaxf(m, a.amax());
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (size_t i = nvec * 16; i < n; ++i) m = fmaxf(m, fabsf(to_f32<T>(x[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane_id() == 0 && m > 0.f) atomicMax(amax_bits, __float_as_uint(m));
}

// Division-free thread -> (row, 16-element chunk) mapping shared by the row-wise quantisers.
// A block of 256 threads covers `rows_per_block` rows x 2^log2_cp chunk slots (slots past the
// row's real chunk count idle); rows longer than 256 chunks take several blocks along grid.y.
struct RowMap {
    int log2_cp;          // chunk slots per row inside a block (power of two, <= 256)
    int rows_per_block;   // 256 >> log2_cp
};
static inline RowMap make_row_map(long long cols, int min_log2) {
    const long long cpr = cols / 16;
    int l = min_log2;
    while ((1ll << l) < cpr && l < 8) ++l;
    RowMap m;
    m.log2_cp = l;
    m.rows_per_block = 256 >> l;
    return m;
}
static inline dim3 row_map_grid(const RowMap& m, long long rows, long long cols) {
    const long long cpr = cols / 16;
    return dim3(static_cast<unsigned>((rows + m.rows_per_block - 1) / m.rows_per_block),
                static_cast<unsigned>((cpr + 255) / 256));
}

// ---- FP8 ---------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
quant_fp8_tensor_kernel(const T* __restrict__ x, size_t n, const uint32_t* amax_bits, float* scale_io,
                        uint8_t* __restrict__ q) {
    griddep_launch_dependents();
    float s;
    if (amax_bits != nullptr) {
        s = fp8_scale_from_amax(__uint_as_float(*amax_bits));
        if (blockIdx.x == 0 && threadIdx.x == 0) *scale_io = s;
    } else {
        s = *scale_io;
    }
    const size_t nvec = n / 16;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        float v[16];
        load16<T>(x + i * 16, v);
        *reinterpret_cast<uint4*>(q + i * 16) = amax_bits != nullptr ? quant16_e4m3<false>(v, s) : quant16_e4m3<true>(v, s);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (size_t i = nvec * 16; i < n; ++i)
            q[i] = static_cast<uint8_t>(cvt_e4m3x2(__fdiv_rn(to_f32<T>(x[i]), s), 0.f) & 0xFFu);
}

// 1 x 128 groups along K: 8 threads per group, 16 elements each.  K % 16 == 0.
template <typename T>
__global__ void __launch_bounds__(256)
quant_fp8_1x128_kernel(const T* __restrict__ x, long long M, int K, uint8_t* __restrict__ q,
                       float* __restrict__ scales, int log2_cp, bool wide) {
    griddep_launch_dependents();   // the GEMM that follows may set itself up now; it waits before reading q / scales
    const int cpr = K / 16;
    const int ng = (K + 127) / 128;
    const long long row = blockIdx.x * static_cast<long long>(256 >> log2_cp) + (threadIdx.x >> log2_cp);
    const int kc = blockIdx.y * 256 + (threadIdx.x & ((1 << log2_cp) - 1));
    const bool valid = row < M && kc < cpr;
    const size_t off = static_cast<size_t>(row) * K + static_cast<size_t>(kc) * 16;
    Chunk16<T> ch;
    if (valid) ch.load(x + off, wide); else ch.zero();
    float m = ch.amax();   // the 8 lanes of a group are adjacent (slots per row are a multiple of 8)
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 4));
    const float s = fp8_scale_from_amax(m);
    if (valid) {
        float v[16];
        ch.to_float(v);
        *reinterpret_cast<uint4*>(q + off) = quant16_e4m3<false>(v, s);
        if ((kc & 7) == 0) scales[static_cast<size_t>(row) * ng + (kc >> 3)] = s;
    }
}

// 128 x 128 blocks of a K-major [N, K] weight: one CTA per block, 64 elements per thread.
template <typename T>
__global__ void __launch_bounds__(256)
quant_fp8_block128_kernel(const T* __restrict__ w, int N, int K, uint8_t* __restrict__ q,
                          float* __restrict__ scales) {
    __shared__ float red[8];
    const int kb = blockIdx.x, nb = blockIdx.y;
    const int r = nb * 128 + (threadIdx.x >> 1);
    const int k0 = kb * 128 + (threadIdx.x & 1) * 64;
    float v[4][16];
    float m = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[c][i] = 0.f;
        if (r < N && k0 + c * 16 < K) load16<T>(w + static_cast<size_t>(r) * K + k0 + c * 16, v[c]);
        m = fmaxf(m, amax16(v[c]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane_id() == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    const float s = fp8_scale_from_amax(m);
    if (threadIdx.x == 0) scales[static_cast<size_t>(nb) * gridDim.x + kb] = s;
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (r < N && k0 + c * 16 < K)
            *reinterpret_cast<uint4*>(q + static_cast<size_t>(r) * K + k0 + c * 16) = quant16_e4m3<false>(v[c], s);
}

// ---- FP4 ---------------------------------------------------------------------------------
constexpr int kMaxGroups = 1024;

// Block scale of one NVFP4 chunk: byte = ue4m3(min((amax16 / 6) / gs, 448)), inv = 1 / (f32(byte) * gs), 0 when that
// product is below FLT_MIN.  The two IEEE divisions are done without dividing: m / 6 as RN(m * RN(1/6)) plus one
// residual correction (exhaustively equal to the division for every m >= 2^-100), a / gs with the reciprocal of gs
// (computed once per thread) and two corrections (Markstein: correctly rounded).  Residuals are exact unless they
// underflow; with gs inside [2^-64, 2^64] that needs a quotient below 2^-36, far under the smallest rounding boundary of
// the scale byte (2^-10), where both forms give byte 0.  An infinite m turns into NaN and fminf returns 448 for it, as
// it does for the infinite quotient.  Other global scales (a caller may give anything) take the real divisions.
struct Nvfp4Scaler {
    float gs, rgs;
    bool fast;
    __device__ __forceinline__ void init(float g) {
        gs = g;
        fast = g >= 0x1p-64f && g <= 0x1p64f;
        rgs = fast ? __frcp_rn(g) : 0.f;
    }
    __device__ __forceinline__ uint32_t operator()(float m, float& inv) const {
        float t;
        if (fast) {
            constexpr float r6 = 0x1.555556p-3f;                           // RN(1/6)
            const float a0 = __fmul_rn(m, r6);
            const float a = __fmaf_rn(__fmaf_rn(-a0, 6.0f, m), r6, a0);      // m / 6
            const float q0 = __fmul_rn(a, rgs);
            const float q1 = __fmaf_rn(__fmaf_rn(-q0, gs, a), rgs, q0);
            t = __fmaf_rn(__fmaf_rn(-q1, gs, a), rgs, q1);                   // a / gs
        } else {
            t = __fdiv_rn(__fdiv_rn(m, 6.0f), gs);
        }
        t = fminf(t, 448.0f);
        const uint32_t sfb = cvt_e4m3x2(t, 0.f) & 0xFFu;
        const float d = __fmul_rn(e4m3_to_float(sfb), gs);
        inv = d >= FLT_MIN ? __frcp_rn(d) : 0.f;
        return sfb;
    }
};

// Where the scale bytes of a row go.  With ragged row groups every group starts at a fresh 128-row tile (tile index =
// number of 128-row tiles of the groups before it).  The kernels visit rows in ascending or descending order, so the
// group of a row is found by stepping a cursor from the previous row's group (the table is monotone after
// monotone_rows) instead of a binary search per row.
struct SfIndexer {
    const int* offs;   // shared-memory copy of the group offsets [G+1], or nullptr
    const int* tile0;  // shared-memory first tile of each group [G+1]
    int groups;
    int katoms;
    int g;             // cursor
    // Byte offset of K-block 0 of `row`, or -1 for a row in front of the first group (it belongs to no group).
    // K-block b of the row is (b >> 2) * 512 + (b & 3) bytes further on.
    __device__ __forceinline__ long long row_base(unsigned row) {
        unsigned tile, rin;
        if (offs == nullptr) {
            tile = row >> 7;
            rin = row & 127u;
        } else {
            const int r = static_cast<int>(row);
            while (g + 1 < groups && r >= offs[g + 1]) ++g;
            while (g > 0 && r < offs[g]) --g;
            const int rl = r - offs[g];
            if (rl < 0) return -1;
            tile = static_cast<unsigned>(tile0[g] + (rl >> 7));
            rin = static_cast<unsigned>(rl) & 127u;
        }
        return static_cast<long long>(static_cast<size_t>(tile) * katoms * 512 + (rin & 31u) * 16 + (rin >> 5) * 4);
    }
};

// All threads: fills the shared tables from the (untrusted, device-resident) group offsets, sanitised exactly as the
// GEMM kernels do, so that both derive the same scale tiles.  Contains two __syncthreads() when offsets are given.
__device__ __forceinline__ void sf_indexer_init(SfIndexer& sfi, int* s_offs, int* s_tile0, const int* group_offsets,
                                                int num_groups, int m_total, int nblk, bool from_the_end) {
    sfi.katoms = (nblk + 3) / 4;
    sfi.groups = num_groups;
    sfi.offs = nullptr;
    sfi.tile0 = nullptr;
    sfi.g = 0;
    if (group_offsets == nullptr) return;
    load_group_offsets(s_offs, group_offsets, num_groups, m_total);
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int g = 0; g < num_groups; ++g) {
            s_tile0[g] = t;
            t += (monotone_rows(s_offs, g) + 127) >> 7;
        }
        s_tile0[num_groups] = t;
    }
    __syncthreads();
    sfi.offs = s_offs;
    sfi.tile0 = s_tile0;
    sfi.g = from_the_end ? num_groups - 1 : 0;
}

// One thread per 16-element chunk; a block of 256 threads covers 2^(8 - log2_cp) rows x 2^log2_cp chunk slots and walks the
// row blocks grid-stride.  Everything that depends only on the thread's column (pointers, scale-tile column, writer role)
// is set up once; per row block there is one 32 x 32 -> 64 bit multiply for the addresses.  These kernels are bound by
// instruction issue as much as by DRAM (ncu: issue slots 81 % busy at 52 % of the DRAM peak before this form), so
// instructions per chunk are what counts.
template <typename T, int FMT>   // FMT 0: NVFP4 (block 16, UE4M3 + global scale)  1: MXFP4 (block 32, E8M0)
__global__ void __launch_bounds__(256)
quant_fp4_kernel(const T* __restrict__ x, unsigned M, int K, float* __restrict__ gs_ptr,
                 const uint32_t* __restrict__ amax_bits, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const int* __restrict__ group_offsets,
                 int num_groups, int log2_cp, unsigned row_blocks, bool wide) {
    griddep_launch_dependents();   // a GEMM that opted in may set itself up (and stream its weight) from now on
    __shared__ int s_offs[kMaxGroups + 1];
    __shared__ int s_tile0[kMaxGroups + 1];
    // After an amax pass the END of the tensor is what the L2 still holds (that pass walks it front to
    // back), so this pass then walks the row blocks back to front and finds much of its input there.
    const bool backwards = FMT == 0 && amax_bits != nullptr;
    SfIndexer sfi;
    sf_indexer_init(sfi, s_offs, s_tile0, group_offsets, num_groups, static_cast<int>(M > 0x7FFFFFFFu ? 0x7FFFFFFFu : M),
                    FMT == 0 ? K / 16 : K / 32, backwards);
    // NVFP4 global scale: given (gs_ptr holds it) or derived here from the tensor amax and published
    Nvfp4Scaler scaler;
    if (FMT == 0) {
        float gs;
        if (amax_bits != nullptr) {
            const float a = __uint_as_float(*amax_bits);
            gs = a == 0.f ? 1.0f : __fdiv_rn(a, 2688.0f);
            if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *gs_ptr = gs;
        } else {
            gs = *gs_ptr;
        }
        scaler.init(gs);
    }
    const int cpr = K >> 4;   // 16-element chunks per row
    const int kc = blockIdx.y * 256 + (threadIdx.x & ((1 << log2_cp) - 1));
    const unsigned rsub = threadIdx.x >> log2_cp;
    const int rpb_log2 = 8 - log2_cp;
    const bool col_ok = kc < cpr;
    const size_t pitch_x = static_cast<size_t>(K) * sizeof(T);
    const size_t pitch_q = static_cast<size_t>(K >> 1);
    const uint8_t* xcol = reinterpret_cast<const uint8_t*>(x) + static_cast<size_t>(kc) * (16 * sizeof(T));
    uint8_t* qcol = q + static_cast<size_t>(kc) * 8;
    // Scale bytes: four consecutive K-blocks of a row are four consecutive bytes of the tile
    // layout, so when the row length allows it one lane stores all four as a word.
    constexpr int LANES_PER_BLK = FMT == 0 ? 1 : 2;
    const int blk = FMT == 0 ? kc : kc >> 1;
    const bool packed = (cpr % (4 * LANES_PER_BLK)) == 0;   // uniform over the grid
    const bool sf_writer = col_ok && (packed ? (kc % (4 * LANES_PER_BLK)) == 0 : (FMT == 0 || (kc & 1) == 0));
    uint8_t* sfcol = sf + static_cast<size_t>(blk >> 2) * 512 + (blk & 3);
    for (unsigned it = blockIdx.x; it < row_blocks; it += gridDim.x) {
        const unsigned rb = backwards ? row_blocks - 1 - it : it;
        const unsigned row = (rb << rpb_log2) + rsub;
        const bool valid = col_ok && row < M;
        Chunk16<T> ch;
        if (valid) ch.load(reinterpret_cast<const T*>(xcol + row * pitch_x), wide); else ch.zero();
        float m = ch.amax();
        float inv;
        uint32_t sfb;
        if (FMT == 0) {
            sfb = scaler(m, inv);
        } else {
            m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));   // cpr is even, so lane pairs share a row
            int e = static_cast<int>((__float_as_uint(m) >> 23) & 0xFFu) - 129;
            e = e < -127 ? -127 : e;
            sfb = static_cast<uint32_t>(e + 127);
            inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
        }
        if (valid) *reinterpret_cast<uint2*>(qcol + row * pitch_q) = ch.quant_e2m1(inv);
        if (packed) {
            uint32_t word = sfb;
            word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 1 * LANES_PER_BLK) << 8;
            word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 2 * LANES_PER_BLK) << 16;
            word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 3 * LANES_PER_BLK) << 24;
            sfb = word;
        }
        if (sf_writer && row < M) {
            const long long base = sfi.row_base(row);
            if (base >= 0) {
                if (packed) *reinterpret_cast<uint32_t*>(sfcol + base) = sfb;
                else sfcol[base] = static_cast<uint8_t>(sfb);
            }
        }
    }
}


// NVFP4 with one global scale PER ROW (per token): gs[m] = amax_row[m] / 2688.  A row's quantisation then depends on
// that row only, so amax, global scale, block scales, nibbles and scale tiles come out of ONE pass: a CTA takes ROWS rows
// at a time (grid-stride), every thread keeps its chunks of those rows in registers while the row maxima are reduced
// through shared memory, then quantises them.  R = chunks per thread and row (row length up to R * 4096 elements).
template <typename T, int R, int ROWS>
__global__ void __launch_bounds__(256)
quant_nvfp4_token_kernel(const T* __restrict__ x, long long M, int K, float* __restrict__ gs_out, uint8_t* __restrict__ q,
                         uint8_t* __restrict__ sf, const int* __restrict__ group_offsets, int num_groups, bool wide) {
    griddep_launch_dependents();
    __shared__ int s_offs[kMaxGroups + 1];
    __shared__ int s_tile0[kMaxGroups + 1];
    __shared__ float red[2][ROWS][8];
    const int cpr = K / 16;
    SfIndexer sfi;
    sf_indexer_init(sfi, s_offs, s_tile0, group_offsets, num_groups, static_cast<int>(M), cpr, false);
    const bool packed = (cpr % 4) == 0;     // four consecutive K-blocks of a row are one word of the tile layout
    const long long row_groups = (M + ROWS - 1) / ROWS;
    int it = 0;
    for (long long rg = blockIdx.x; rg < row_groups; rg += gridDim.x, ++it) {
        const long long row0 = rg * ROWS;
        Chunk16<T> ch[ROWS][R];
        float bm[ROWS][R];
        float m[ROWS];
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            m[j] = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int kc = threadIdx.x + r * 256;
                if (row0 + j < M && kc < cpr) ch[j][r].load(x + (static_cast<size_t>(row0 + j) * cpr + kc) * 16, wide);
                else ch[j][r].zero();
            }
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                bm[j][r] = ch[j][r].amax();
                m[j] = fmaxf(m[j], bm[j][r]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m[j] = fmaxf(m[j], __shfl_xor_sync(0xFFFFFFFFu, m[j], o));
            if (lane_id() == 0) red[it & 1][j][threadIdx.x >> 5] = m[j];
        }
        __syncthreads();     // the other buffer is written next time: nobody can still be reading it then
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const long long row = row0 + j;
            float a = red[it & 1][j][0];
#pragma unroll
            for (int w = 1; w < 8; ++w) a = fmaxf(a, red[it & 1][j][w]);
            const float gs = a == 0.f ? 1.0f : __fdiv_rn(a, 2688.0f);
            if (threadIdx.x == 0 && row < M) gs_out[row] = gs;
            Nvfp4Scaler scaler;
            scaler.init(gs);
            // rows come in ascending order (the cursor of the indexer relies on it); only the lanes that store need it
            const long long base = row < M ? sfi.row_base(static_cast<unsigned>(row)) : -1;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int kc = threadIdx.x + r * 256;
                const bool valid = row < M && kc < cpr;
                float inv;
                uint32_t sfb = scaler(bm[j][r], inv);
                if (valid) *reinterpret_cast<uint2*>(q + (static_cast<size_t>(row) * cpr + kc) * 8) = ch[j][r].quant_e2m1(inv);
                uint8_t* dst = sf + base + static_cast<size_t>(kc >> 2) * 512 + (kc & 3);
                if (packed) {
                    uint32_t word = sfb;
                    word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 1) << 8;
                    word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 2) << 16;
                    word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 3) << 24;
                    if (valid && base >= 0 && (kc & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = word;
                } else if (valid && base >= 0) {
                    *dst = static_cast<uint8_t>(sfb);
                }
            }
        }
    }
}

// The same per-token quantiser with ONE WARP per row, for bf16 rows of up to 4096 elements (R = chunks per lane, row
// length up to R * 512): the row maximum needs only shuffles - no shared memory, no block barrier - so the warps of a CTA
// run independently and the loads of many rows are in flight per SM.  The CTA-per-row form above spends most of a short
// row's time in its two barriers (131072 rows of 4096: 0.49 ms, 2.8 TB/s).
template <int R>
__global__ void __launch_bounds__(256)
quant_nvfp4_token_warp_kernel(const __nv_bfloat16* __restrict__ x, long long M, int K, float* __restrict__ gs_out,
                              uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const int* __restrict__ group_offsets,
                              int num_groups, bool wide) {
    griddep_launch_dependents();
    __shared__ int s_offs[kMaxGroups + 1];
    __shared__ int s_tile0[kMaxGroups + 1];
    const int cpr = K / 16;
    SfIndexer sfi;
    sf_indexer_init(sfi, s_offs, s_tile0, group_offsets, num_groups, static_cast<int>(M), cpr, false);
    const bool packed = (cpr % 4) == 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row_blocks = (M + 7) / 8;
    for (long long rb = blockIdx.x; rb < row_blocks; rb += gridDim.x) {
        const long long row = rb * 8 + warp;               // ascending per warp: the indexer's cursor relies on it
        const bool row_ok = row < M;
        Chunk16<__nv_bfloat16> ch[R];
        float bm[R];
        float m = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int kc = lane + 32 * r;
            if (row_ok && kc < cpr) ch[r].load(x + (static_cast<size_t>(row) * cpr + kc) * 16, wide);
            else ch[r].zero();
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            bm[r] = ch[r].amax();
            m = fmaxf(m, bm[r]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        const float gs = m == 0.f ? 1.0f : __fdiv_rn(m, 2688.0f);
        if (lane == 0 && row_ok) gs_out[row] = gs;
        Nvfp4Scaler scaler;
        scaler.init(gs);
        const long long base = row_ok ? sfi.row_base(static_cast<unsigned>(row)) : -1;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int kc = lane + 32 * r;
            const bool valid = row_ok && kc < cpr;
            float inv;
            const uint32_t sfb = scaler(bm[r], inv);
            if (valid) *reinterpret_cast<uint2*>(q + (static_cast<size_t>(row) * cpr + kc) * 8) = ch[r].quant_e2m1(inv);
            uint8_t* dst = sf + base + static_cast<size_t>(kc >> 2) * 512 + (kc & 3);
            if (packed) {
                uint32_t word = sfb;
                word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 1) << 8;
                word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 2) << 16;
                word |= __shfl_down_sync(0xFFFFFFFFu, sfb, 3) << 24;
                if (valid && base >= 0 && (kc & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = word;
            } else if (valid && base >= 0) {
                *dst = static_cast<uint8_t>(sfb);
            }
        }
    }
}

// Small tensors (decode: a handful of activation rows): tensor amax, global scale and the NVFP4
// quantisation in ONE launch of a single CTA, instead of memset + amax + scale + quantise.
template <typename T>
__global__ void __launch_bounds__(1024)
quant_nvfp4_small_kernel(const T* __restrict__ x, int M, int K, float* __restrict__ gs_out,
                         uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
    griddep_launch_dependents();
    __shared__ float red[32];
    __shared__ float s_gs;
    const int cpr = K / 16;
    const int total = M * cpr;
    float m = 0.f;
    for (int c = threadIdx.x; c < total; c += blockDim.x) {
        float v[16];
        load16<T>(x + static_cast<size_t>(c) * 16, v);
        m = fmaxf(m, amax16(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane_id() == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.f;
        for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) a = fmaxf(a, red[i]);
        s_gs = a == 0.f ? 1.0f : __fdiv_rn(a, 2688.0f);
        *gs_out = s_gs;
    }
    __syncthreads();
    Nvfp4Scaler scaler;
    scaler.init(s_gs);
    const int katoms = (cpr + 3) / 4;
    for (int c = threadIdx.x; c < total; c += blockDim.x) {
        const int row = c / cpr, kc = c - row * cpr;
        float v[16];
        load16<T>(x + static_cast<size_t>(c) * 16, v);   // second read comes from L1/L2
        float inv;
        const uint32_t sfb = scaler(amax16(v), inv);
        *reinterpret_cast<uint2*>(q + static_cast<size_t>(c) * 8) = quant16_e2m1(v, inv);
        sf[(static_cast<size_t>(row >> 7) * katoms + (kc >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kc & 3)] =
            static_cast<uint8_t>(sfb);
    }
}

// Up to 256 K elements (decode batches; at 1 M elements the eight SMs of the cluster were measured slower than the
// three-launch path that uses the whole GPU: 30.8 against 27.6 us for the 128 x 8192 step): the same single launch, spread over
// one cluster of eight CTAs.  Each CTA reduces its share, the eight maxima meet through
// distributed shared memory at a cluster barrier, and every CTA then quantises its share (second
// read from L1/L2).  The padding bytes of the scale tiles are zeroed here too, so this path
// needs no memset and no scratch word.
constexpr int kQuantClusterCtas = 8;
__device__ __forceinline__ float ld_cluster_f32(const float* local_ptr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
template <typename T>
__global__ void __cluster_dims__(kQuantClusterCtas, 1, 1) __launch_bounds__(1024)
quant_nvfp4_cluster_kernel(const T* __restrict__ x, int M, int K, float* __restrict__ gs_out,
                           uint8_t* __restrict__ q, uint8_t* __restrict__ sf, unsigned sf_clear_vec16) {
    griddep_launch_dependents();
    __shared__ float red[32];
    __shared__ float s_cta_amax;
    __shared__ float s_gs;
    const uint32_t rank = cluster_ctarank();
    const int gtid = static_cast<int>(rank) * 1024 + threadIdx.x;
    constexpr int kThreads = kQuantClusterCtas * 1024;
    for (unsigned i = gtid; i < sf_clear_vec16; i += kThreads) reinterpret_cast<uint4*>(sf)[i] = make_uint4(0u, 0u, 0u, 0u);
    const int cpr = K / 16;
    const int total = M * cpr;
    float m = 0.f;
    for (int c = gtid; c < total; c += kThreads) {
        float v[16];
        load16<T>(x + static_cast<size_t>(c) * 16, v);
        m = fmaxf(m, amax16(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane_id() == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float a = red[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        if (threadIdx.x == 0) s_cta_amax = a;
    }
    cluster_sync_all();     // maxima published; the zeroed scale bytes are ordered before any scale store below
    if (threadIdx.x < 32) {
        float a = threadIdx.x < kQuantClusterCtas ? ld_cluster_f32(&s_cta_amax, threadIdx.x) : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        if (threadIdx.x == 0) {
            s_gs = a == 0.f ? 1.0f : __fdiv_rn(a, 2688.0f);
            if (rank == 0) *gs_out = s_gs;
        }
    }
    __syncthreads();
    // this CTA is done reading its peers; they may not exit before everyone has said so (waited for at the end)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    Nvfp4Scaler scaler;
    scaler.init(s_gs);
    const int katoms = (cpr + 3) / 4;
    for (int c = gtid; c < total; c += kThreads) {
        const int row = c / cpr, kc = c - row * cpr;
        float v[16];
        load16<T>(x + static_cast<size_t>(c) * 16, v);
        float inv;
        const uint32_t sfb = scaler(amax16(v), inv);
        *reinterpret_cast<uint2*>(q + static_cast<size_t>(c) * 8) = quant16_e2m1(v, inv);
        sf[(static_cast<size_t>(row >> 7) * katoms + (kc >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kc & 3)] =
            static_cast<uint8_t>(sfb);
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Per-tensor FP8 of a small tensor (up to 1 M elements, e.g. the 1024 x 1024 plumbing configuration) in ONE launch: the
// same 8-CTA cluster scheme as above - every CTA reduces its share, the maxima meet through distributed shared memory,
// the scale max(amax / 448, 1e-12) is published, and the second sweep (from L2) quantises - instead of memset + amax
// kernel + quantise kernel, whose launch gaps are longer than their work at this size.  n % 16 == 0.
template <typename T>
__global__ void __cluster_dims__(kQuantClusterCtas, 1, 1) __launch_bounds__(1024)
quant_fp8_tensor_cluster_kernel(const T* __restrict__ x, int nvec, float* __restrict__ scale_out, uint8_t* __restrict__ q) {
    griddep_launch_dependents();
    __shared__ float red[32];
    __shared__ float s_cta_amax;
    __shared__ float s_scale;
    const uint32_t rank = cluster_ctarank();
    const int gtid = static_cast<int>(rank) * 1024 + threadIdx.x;
    constexpr int kThreads = kQuantClusterCtas * 1024;
    float m = 0.f;
    for (int c = gtid; c < nvec; c += kThreads) {
        float v[16];
        load16<T>(x + static_cast<size_t>(c) * 16, v);
        m = fmaxf(m, amax16(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane_id() == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float a = red[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        if (threadIdx.x == 0) s_cta_amax = a;
    }
    cluster_sync_all();
    if (threadIdx.x < 32) {
        float a = threadIdx.x < kQuantClusterCtas ? ld_cluster_f32(&s_cta_amax, threadIdx.x) : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        if (threadIdx.x == 0) {
            s_scale = fp8_scale_from_amax(a);
            if (rank == 0) *scale_out = s_scale;
        }
    }
    __syncthreads();
    // this CTA is done reading its peers; they may not exit before everyone has said so (waited for at the end)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const float s = s_scale;
    for (int c = gtid; c < nvec; c += kThreads) {
        float v[16];
        load16<T>(x + static_cast<size_t>(c) * 16, v);
        *reinterpret_cast<uint4*>(q + static_cast<size_t>(c) * 16) = quant16_e4m3<false>(v, s);
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- byte-matrix transpose ([R, C] -> [C, R]), used to turn a [K, N] weight K-major --------
__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                           int R, int C) {
    __shared__ uint8_t tile[64][65];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        int r = i >> 6, c = i & 63;
        tile[r][c] = (r0 + r < R && c0 + c < C) ? in[static_cast<size_t>(r0 + r) * C + c0 + c] : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 64; i += 256) {
        int c = i >> 6, r = i & 63;
        if (r0 + r < R && c0 + c < C) out[static_cast<size_t>(c0 + c) * R + r0 + r] = tile[r][c];
    }
}

// ---- host launchers ------------------------------------------------------------------------
static inline int grid_for(size_t work_items, int per_block, int cap) {
    size_t g = (work_items + per_block - 1) / per_block;
    if (g < 1) g = 1;
    return static_cast<int>(g > static_cast<size_t>(cap) ? cap : g);
}

template <typename T>
static cudaError_t quant_fp8_typed(const T* x, long long rows, long long cols, int mode, float* scale_io,
                                   int scale_given, uint8_t* q, uint32_t* ws, cudaStream_t st) {
    const size_t n = static_cast<size_t>(rows) * cols;
    // 256-bit loads need every 16-element chunk on a 32-byte boundary: base pointer and row pitch
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31u) == 0 && (static_cast<size_t>(cols) * sizeof(T)) % 32 == 0;
    if (mode == DSL_FP8_PER_TENSOR && !scale_given && n % 16 == 0 && n >= (16u << 10) && n <= (1u << 20)) {
        quant_fp8_tensor_cluster_kernel<T><<<kQuantClusterCtas, 1024, 0, st>>>(x, static_cast<int>(n / 16), scale_io, q);
        return cudaGetLastError();
    }
    if (mode == DSL_FP8_PER_TENSOR) {
        const int grid = grid_for(n / 16, 256, 148 * 16);
        if (!scale_given) {
            cudaError_t e = cudaMemsetAsync(ws, 0, 4, st);
            if (e != cudaSuccess) return e;
            amax_kernel<T><<<grid, 256, 0, st>>>(x, n, ws, wide);
        }
        quant_fp8_tensor_kernel<T><<<grid, 256, 0, st>>>(x, n, scale_given ? nullptr : ws, scale_io, q);
    } else if (mode == DSL_FP8_GROUP_1X128) {
        const RowMap rm = make_row_map(cols, 3);
        const dim3 grid = row_map_grid(rm, rows, cols);
        if (grid.x > 0 && grid.y > 0)
            quant_fp8_1x128_kernel<T><<<grid, 256, 0, st>>>(x, rows, static_cast<int>(cols), q, scale_io, rm.log2_cp, wide);
    } else {
        dim3 grid(static_cast<unsigned>((cols + 127) / 128), static_cast<unsigned>((rows + 127) / 128));
        if (grid.x > 0 && grid.y > 0)
            quant_fp8_block128_kernel<T><<<grid, 256, 0, st>>>(x, static_cast<int>(rows), static_cast<int>(cols), q, scale_io);
    }
    return cudaGetLastError();
}

cudaError_t launch_quant_fp8(const void* x, int dtype, long long rows, long long cols, int mode, float* scale_io,
                             int scale_given, uint8_t* q, uint32_t* ws, cudaStream_t st) {
    switch (dtype) {
        case DSL_F32: return quant_fp8_typed(static_cast<const float*>(x), rows, cols, mode, scale_io, scale_given, q, ws, st);
        case DSL_BF16: return quant_fp8_typed(static_cast<const __nv_bfloat16*>(x), rows, cols, mode, scale_io, scale_given, q, ws, st);
        default: return quant_fp8_typed(static_cast<const __half*>(x), rows, cols, mode, scale_io, scale_given, q, ws, st);
    }
}

template <typename T>
static cudaError_t quant_fp4_typed(const T* x, long long rows, long long cols, int format, float* gs_io,
                                   int gs_given, uint8_t* q, uint8_t* sf, size_t sf_bytes, int sf_needs_clear,
                                   const int* group_offsets, int num_groups, uint32_t* ws, cudaStream_t st) {
    const size_t n = static_cast<size_t>(rows) * cols;
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31u) == 0 && (static_cast<size_t>(cols) * sizeof(T)) % 32 == 0;
    cudaError_t e;
    if (format == DSL_FP4_NV && !gs_given && group_offsets == nullptr && n > (32u << 10) && n <= (256u << 10)) {
        const unsigned clear16 = sf_needs_clear ? static_cast<unsigned>(sf_bytes / 16) : 0u;
        quant_nvfp4_cluster_kernel<T><<<kQuantClusterCtas, 1024, 0, st>>>(x, static_cast<int>(rows), static_cast<int>(cols), gs_io, q, sf, clear16);
        return cudaGetLastError();
    }
    if (sf_needs_clear && sf_bytes > 0) {
        e = cudaMemsetAsync(sf, 0, sf_bytes, st);
        if (e != cudaSuccess) return e;
    }
    if (format == DSL_FP4_NV && !gs_given && group_offsets == nullptr && n <= (32u << 10)) {
        quant_nvfp4_small_kernel<T><<<1, 1024, 0, st>>>(x, static_cast<int>(rows), static_cast<int>(cols), gs_io, q, sf);
        return cudaGetLastError();
    }
    if (format == DSL_FP4_NV && !gs_given) {
        e = cudaMemsetAsync(ws, 0, 4, st);
        if (e != cudaSuccess) return e;
        amax_kernel<T><<<grid_for(n / 16, 256, 148 * 8), 256, 0, st>>>(x, n, ws, wide);   // one resident wave
    }
    const uint32_t* amax_bits = (format == DSL_FP4_NV && !gs_given) ? ws : nullptr;
    const RowMap rm = make_row_map(cols, 1);
    dim3 grid = row_map_grid(rm, rows, cols);
    const unsigned row_blocks = grid.x;
    const unsigned cap = 148u * 16u / (grid.y > 0 ? grid.y : 1u) + 1u;   // persistent: a few CTAs per SM
    if (grid.x > cap) grid.x = cap;
    const unsigned m = static_cast<unsigned>(rows);                        // at most 2^31 (checked by the caller)
    if (grid.x > 0 && grid.y > 0) {
        if (format == DSL_FP4_NV)
            quant_fp4_kernel<T, 0><<<grid, 256, 0, st>>>(x, m, static_cast<int>(cols), gs_io, amax_bits, q, sf, group_offsets, num_groups, rm.log2_cp, row_blocks, wide);
        else
            quant_fp4_kernel<T, 1><<<grid, 256, 0, st>>>(x, m, static_cast<int>(cols), nullptr, nullptr, q, sf, group_offsets, num_groups, rm.log2_cp, row_blocks, wide);
    }
    return cudaGetLastError();
}

cudaError_t launch_quant_fp4(const void* x, int dtype, long long rows, long long cols, int format, float* gs_io,
                             int gs_given, uint8_t* q, uint8_t* sf, size_t sf_bytes, int sf_needs_clear,
                             const int* group_offsets, int num_groups, uint32_t* ws, cudaStream_t st) {
    switch (dtype) {
        case DSL_F32: return quant_fp4_typed(static_cast<const float*>(x), rows, cols, format, gs_io, gs_given, q, sf, sf_bytes, sf_needs_clear, group_offsets, num_groups, ws, st);
        case DSL_BF16: return quant_fp4_typed(static_cast<const __nv_bfloat16*>(x), rows, cols, format, gs_io, gs_given, q, sf, sf_bytes, sf_needs_clear, group_offsets, num_groups, ws, st);
        default: return quant_fp4_typed(static_cast<const __half*>(x), rows, cols, format, gs_io, gs_given, q, sf, sf_bytes, sf_needs_clear, group_offsets, num_groups, ws, st);
    }
}

template <typename T>
static cudaError_t quant_token_typed(const T* x, long long rows, long long cols, float* gs_out, uint8_t* q, uint8_t* sf,
                                     const int* group_offsets, int num_groups, cudaStream_t st) {
    const bool wide = (reinterpret_cast<uintptr_t>(x) & 31u) == 0 && (static_cast<size_t>(cols) * sizeof(T)) % 32 == 0;
    const long long cpr = cols / 16;
    const int k = static_cast<int>(cols);
    // One row per CTA and pass (ROWS = 1).  Taking several rows at a time to keep more loads in flight was measured
    // and lost (8192 x 8192: 59 -> 68 us, 131072 x 4096: 563 -> 627 us): the kernel is bound by instruction issue, and
    // the extra registers (128 instead of about 48 per thread) halve the warps that can hide each other's latencies.
    if (sizeof(T) == 2 && !dsl_is_half<T>::value && cpr <= 256) {     // bf16 rows of up to 4096 elements: a warp per row
        const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
        const long long row_blocks = (rows + 7) / 8;
        const unsigned wgrid = static_cast<unsigned>(row_blocks < 148 * 4 ? row_blocks : 148 * 4);
        if (cpr <= 32) quant_nvfp4_token_warp_kernel<1><<<wgrid, 256, 0, st>>>(xb, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
        else if (cpr <= 64) quant_nvfp4_token_warp_kernel<2><<<wgrid, 256, 0, st>>>(xb, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
        else if (cpr <= 128) quant_nvfp4_token_warp_kernel<4><<<wgrid, 256, 0, st>>>(xb, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
        else quant_nvfp4_token_warp_kernel<8><<<wgrid, 256, 0, st>>>(xb, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
        return cudaGetLastError();
    }
    const unsigned grid = static_cast<unsigned>(rows < 148 * 8 ? rows : 148 * 8);
    if (cpr <= 256) quant_nvfp4_token_kernel<T, 1, 1><<<grid, 256, 0, st>>>(x, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
    else if (cpr <= 512) quant_nvfp4_token_kernel<T, 2, 1><<<grid, 256, 0, st>>>(x, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
    else if (cpr <= 1024) quant_nvfp4_token_kernel<T, 4, 1><<<grid, 256, 0, st>>>(x, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
    else quant_nvfp4_token_kernel<T, 8, 1><<<grid, 256, 0, st>>>(x, rows, k, gs_out, q, sf, group_offsets, num_groups, wide);
    return cudaGetLastError();
}

// NVFP4 with per-token global scales; cols <= 32768 (checked by the caller).
cudaError_t launch_quant_nvfp4_per_token(const void* x, int dtype, long long rows, long long cols, float* gs_out, uint8_t* q,
                                         uint8_t* sf, size_t sf_bytes, int sf_needs_clear, const int* group_offsets,
                                         int num_groups, cudaStream_t st) {
    if (sf_needs_clear && sf_bytes > 0) {
        cudaError_t e = cudaMemsetAsync(sf, 0, sf_bytes, st);
        if (e != cudaSuccess) return e;
    }
    switch (dtype) {
        case DSL_F32: return quant_token_typed(static_cast<const float*>(x), rows, cols, gs_out, q, sf, group_offsets, num_groups, st);
        case DSL_BF16: return quant_token_typed(static_cast<const __nv_bfloat16*>(x), rows, cols, gs_out, q, sf, group_offsets, num_groups, st);
        default: return quant_token_typed(static_cast<const __half*>(x), rows, cols, gs_out, q, sf, group_offsets, num_groups, st);
    }
}

cudaError_t launch_transpose_u8(const uint8_t* in, uint8_t* out, int R, int C, cudaStream_t st) {
    dim3 grid((C + 63) / 64, (R + 63) / 64);
    if (grid.x > 0 && grid.y > 0) transpose_u8_kernel<<<grid, 256, 0, st>>>(in, out, R, C);
    return cudaGetLastError();
}

}  // namespace dsl
