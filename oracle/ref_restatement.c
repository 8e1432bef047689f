/*
 * Host restatement of the reference's CUDA emulation kernels on the quantised-GEMM
 * path, written as plain C loops.  TEST INFRASTRUCTURE ONLY: it is the checker for
 * the numpy oracle and the CUDA kernels, never part of the shipped library.
 *
 * Each function names the reference kernel it restates.  Where the CUDA compiler
 * contracts `acc += a * b` into a fused multiply-add, fmaf() is written out so the
 * rounding sequence is the same as the device code built without fast-math.
 * Build with -ffp-contract=off so nothing else is fused.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

static const float E2M1_LUT[16] = {          /* cuda/gemm/fp4_gemm.cu:30-33 */
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* fp32 -> E4M3, round-to-nearest-even, saturate to +-448, NaN -> 0x7F: the
 * conversion `__nv_fp8_e4m3(float)` performs at cuda/gemm/fp8_gemm.cu:142. */
uint8_t rs_e4m3_from_float(float x) {
    uint32_t b;
    memcpy(&b, &x, 4);
    uint8_t sign = (uint8_t)((b >> 24) & 0x80u);
    uint32_t ab = b & 0x7FFFFFFFu;
    if (ab > 0x7F800000u) return 0x7F;
    float a;
    memcpy(&a, &ab, 4);
    if (a > 448.0f) a = 448.0f;
    memcpy(&ab, &a, 4);
    uint32_t code;
    if (a < 0.015625f) {                       /* below 2^-6: subnormal grid of 2^-9 */
        code = (uint32_t)nearbyint((double)a * 512.0);
    } else {
        uint32_t r = ab + 0x7FFFFu + ((ab >> 20) & 1u);
        code = (r >> 20) - ((127u - 7u) << 3);
    }
    if (code > 0x7Eu) code = 0x7Eu;
    return (uint8_t)(code | sign);
}

float rs_e4m3_to_float(uint8_t v) {
    int e = (v >> 3) & 0xF, m = v & 7;
    float s = (v & 0x80) ? -1.0f : 1.0f;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) return s * (float)m * 0.001953125f;
    return s * ldexpf(1.0f + (float)m / 8.0f, e - 7);
}

/* cuda/gemm/fp8_gemm.cu:119-144 (quantize_to_fp8_kernel) */
void rs_quantize_fp8(const float* in, uint8_t* out, float* scale_out, long n) {
    float amax = 0.0f;
    for (long i = 0; i < n; i++) amax = fmaxf(amax, fabsf(in[i]));
    float scale = amax / 448.0f;
    if (scale < 1e-12f) scale = 1e-12f;
    *scale_out = scale;
    for (long i = 0; i < n; i++) out[i] = rs_e4m3_from_float(in[i] / scale);
}

/* cuda/gemm/fp8_gemm.cu:29-65 (fp8_gemm_per_tensor_kernel): operands are
 * dequantised BEFORE the product; B is [K, N] row-major. */
void rs_fp8_gemm_per_tensor(const uint8_t* A, const uint8_t* B, float* C,
                            int M, int N, int K, float sa, float sb) {
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) {
                float a = rs_e4m3_to_float(A[(size_t)m * K + k]) * sa;
                float b = rs_e4m3_to_float(B[(size_t)k * N + n]) * sb;
                acc = fmaf(a, b, acc);
            }
            C[(size_t)m * N + n] = acc;
        }
}

/* cuda/gemm/fp8_gemm.cu:69-99 (fp8_gemm_groupwise_kernel): sa [M, ng], sb [ng, N]. */
void rs_fp8_gemm_groupwise(const uint8_t* A, const uint8_t* B, float* C,
                           int M, int N, int K, int G, const float* sa, const float* sb) {
    int ng = (K + G - 1) / G;
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int g = 0; g < ng; g++) {
                int k1 = (g + 1) * G < K ? (g + 1) * G : K;
                float ga = 0.0f;
                for (int k = g * G; k < k1; k++)
                    ga = fmaf(rs_e4m3_to_float(A[(size_t)m * K + k]),
                              rs_e4m3_to_float(B[(size_t)k * N + n]), ga);
                acc = fmaf(ga * sa[(size_t)m * ng + g], sb[(size_t)g * N + n], acc);
            }
            C[(size_t)m * N + n] = acc;
        }
}

/* cuda/gemm/fp4_gemm.cu:50-90 (quantize_fp32_to_nvfp4): flat buffer, 32 per block,
 * fp32 scale = max(amax/6, 1e-12), v = x * (1/scale), first-minimum LUT search. */
void rs_quantize_fp4(const float* in, uint8_t* out, float* scales, long n) {
    long nb = (n + 31) / 32;
    for (long b = 0; b < nb; b++) {
        long start = b * 32, end = start + 32 < n ? start + 32 : n;
        float amax = 0.0f;
        for (long i = start; i < end; i++) amax = fmaxf(amax, fabsf(in[i]));
        float scale = amax / 6.0f;
        if (scale < 1e-12f) scale = 1e-12f;
        scales[b] = scale;
        float inv = 1.0f / scale;
        for (long i = start; i < end; i += 2) {
            float v0 = in[i] * inv;
            float v1 = (i + 1 < end) ? in[i + 1] * inv : 0.0f;
            uint8_t q0 = 0, q1 = 0;
            float e0 = 1e30f, e1 = 1e30f;
            for (int j = 0; j < 16; j++) {
                float d0 = fabsf(E2M1_LUT[j] - v0), d1 = fabsf(E2M1_LUT[j] - v1);
                if (d0 < e0) { e0 = d0; q0 = (uint8_t)j; }
                if (d1 < e1) { e1 = d1; q1 = (uint8_t)j; }
            }
            out[i / 2] = (uint8_t)((q1 << 4) | q0);
        }
    }
}

/* cuda/gemm/fp4_gemm.cu:95-137 (fp4_gemm_kernel): A packed [M,K] (pairs along K),
 * B packed [K,N] (pairs along N), sa [M, K/32], sb [K/32, N]. */
void rs_fp4_gemm(const uint8_t* A, const uint8_t* B, float* C,
                 const float* sa, const float* sb, int M, int N, int K) {
    int ng = (K + 31) / 32;
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int g = 0; g < ng; g++) {
                int k1 = g * 32 + 32 < K ? g * 32 + 32 : K;
                float ga = 0.0f;
                for (int k = g * 32; k < k1; k++) {
                    size_t ai = (size_t)m * K + k, bi = (size_t)k * N + n;
                    uint8_t an = (ai & 1) ? (A[ai / 2] >> 4) : (A[ai / 2] & 0xF);
                    uint8_t bn = (bi & 1) ? (B[bi / 2] >> 4) : (B[bi / 2] & 0xF);
                    ga = fmaf(E2M1_LUT[an], E2M1_LUT[bn], ga);
                }
                acc = fmaf(ga * sa[(size_t)m * ng + g], sb[(size_t)g * N + n], acc);
            }
            C[(size_t)m * N + n] = acc;
        }
}

/* cuda/gemm/grouped_gemm.cu:27-32 (GemmProblem; offsets count ELEMENTS) */
typedef struct { int M, N, K, A_offset, B_offset, C_offset; } rs_gemm_problem;

/* cuda/gemm/grouped_gemm.cu:79-104 (grouped_gemm_variable_kernel) */
void rs_grouped_gemm_variable(const float* A, const float* B, float* C,
                              const rs_gemm_problem* p, int groups) {
    for (int g = 0; g < groups; g++) {
        const float* a = A + p[g].A_offset;
        const float* b = B + p[g].B_offset;
        float* c = C + p[g].C_offset;
        for (int m = 0; m < p[g].M; m++)
            for (int n = 0; n < p[g].N; n++) {
                float acc = 0.0f;
                for (int k = 0; k < p[g].K; k++)
                    acc = fmaf(a[(size_t)m * p[g].K + k], b[(size_t)k * p[g].N + n], acc);
                c[(size_t)m * p[g].N + n] = acc;
            }
    }
}

/* cuda/gemm/grouped_gemm.cu:36-75 (grouped_gemm_fixed_kernel): [G,M,K] x [G,K,N] */
void rs_grouped_gemm_fixed(const float* A, const float* B, float* C,
                           int M, int N, int K, int groups) {
    for (int g = 0; g < groups; g++)
        for (int m = 0; m < M; m++)
            for (int n = 0; n < N; n++) {
                float acc = 0.0f;
                for (int k = 0; k < K; k++)
                    acc = fmaf(A[((size_t)g * M + m) * K + k], B[((size_t)g * K + k) * N + n], acc);
                C[((size_t)g * M + m) * N + n] = acc;
            }
}
