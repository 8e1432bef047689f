/* Test infrastructure (not part of the product): brute-force check that the division-free quotient used by the
 * E4M3 quantisers (dsl_tool_b200/csrc/quant.cu, div2_for_e4m3) equals the IEEE quotient x / s.
 *
 *   y  = RN(1 / s)                       one reciprocal per 16 elements on the GPU
 *   q0 = RN(x * y)
 *   q1 = RN(q0 + RN(x - q0 * s) * y)     residual by FMA, exact
 *   q2 = RN(q1 + RN(x - q1 * s) * y)     Markstein: correctly rounded
 *   a zero or infinite q0 is returned as it is
 *
 * Scales are what the quantisers produce: s = max(amax / 448, 1e-12) for an amax that bounds |x|.  Quotients
 * below 2^-11 are only required to stay below the smallest E4M3 rounding boundary, 2^-10 (there the residual may
 * underflow and both values convert to zero).
 *
 * A caller may also GIVE the scale (dsl_quant_fp8 with scale_given): then it can be far below 1e-12, its
 * reciprocal can overflow and the residual argument no longer holds, so the quantiser uses the corrected
 * quotient only for scales inside [1e-12, 3e38] and a real division otherwise.  Mode 2 checks that rule over
 * scales drawn from the whole fp32 range (subnormals included) against dividends of any magnitude.
 *
 * Mode 3 checks the NVFP4 block scale the same way (Nvfp4Scaler in quant.cu): t = min((m / 6) / gs, 448) with
 * m / 6 = RN(m * RN(1/6)) + one correction and a / gs = RN(a * RN(1/gs)) + two corrections, for global scales inside
 * [2^-64, 2^64] (others divide for real on the GPU), block maxima m of every bf16 value and random fp32 values up to
 * the tensor maximum 2688 * gs and beyond, and m = Inf.  t below 2^-11 must only stay below 2^-10 (scale byte 0).
 * Mode 4 is the exhaustive statement behind the single correction for the constant divisors: for EVERY float m in
 * [2^-100, FLT_MAX], RN(m * r) corrected once equals m / d for d = 6, 448 and 2688 (about 80 s; not part of the tests'
 * default run).
 *
 * usage: quotient_check <scales> <mode>    mode 0: every bf16 dividend up to amax; mode 1: random fp32 dividends;
 *                                          mode 2: given scales of any size, random dividends;
 *                                          mode 3: NVFP4 block scale; mode 4: constant divisors, exhaustive
 * prints "checked N mismatches M" and exits 0 when M == 0.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static uint64_t rs = 88172645463325252ull;
static uint64_t rnd(void) { rs ^= rs << 13; rs ^= rs >> 7; rs ^= rs << 17; return rs; }
static float from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static float quotient(float x, float s, float y) {
    const float q0 = x * y;
    const float q1 = fmaf(fmaf(-q0, s, x), y, q0);
    const float q2 = fmaf(fmaf(-q1, s, x), y, q1);
    return (q0 + q0 == q0) ? q0 : q2;
}

/* what quant16_e4m3 computes for one element */
static float quotient_guarded(float x, float s) {
    if (s >= 1e-12f && s <= 3.0e38f) return quotient(x, s, 1.0f / s);
    return x / s;
}

/* what Nvfp4Scaler computes before the E4M3 conversion */
static float block_scale_fast(float m, float gs, float rgs) {
    const float r6 = 0x1.555556p-3f;
    const float a0 = m * r6;
    const float a = fmaf(fmaf(-a0, 6.0f, m), r6, a0);
    const float q0 = a * rgs;
    const float q1 = fmaf(fmaf(-q0, gs, a), rgs, q0);
    const float t = fmaf(fmaf(-q1, gs, a), rgs, q1);
    return fminf(t, 448.0f);
}
static float block_scale_plain(float m, float gs) { return fminf((m / 6.0f) / gs, 448.0f); }

static long checked = 0, bad = 0;
static void check_block_scale(float m, float gs, float rgs) {
    const float want = block_scale_plain(m, gs);
    const float got = block_scale_fast(m, gs, rgs);
    if (want < 0x1p-11f) {
        if (!(got < 0x1p-10f) || got < 0.0f) ++bad;
    } else if (memcmp(&got, &want, 4) != 0) {
        ++bad;
    }
    ++checked;
}
static void check(float x, float s, float y) {
    const float want = x / s;
    const float got = quotient(x, s, y);
    if (fabsf(want) < 0x1p-11f) {
        if (!(fabsf(got) < 0x1p-10f) || signbit(got) != signbit(want)) ++bad;
    } else if (memcmp(&got, &want, 4) != 0) {
        ++bad;
    }
    ++checked;
}

int main(int argc, char** argv) {
    const long scales = argc > 1 ? atol(argv[1]) : 200;
    const int mode = argc > 2 ? atoi(argv[2]) : 0;
    if (mode == 3) {
        for (long it = 0; it < scales; ++it) {
            /* global scales: amax / 2688 of a bf16 or fp32 amax of ordinary size, or anything inside the guard */
            float gs;
            if (it % 3 == 0) gs = from_bits((uint32_t)(0x1F800000u + rnd() % (0x5F800000u - 0x1F800000u)));   /* 2^-64 .. 2^64 */
            else {
                uint32_t ab = (uint32_t)(0x30000000u + rnd() % 0x20000000u);
                if (it & 1) ab &= 0xFFFF0000u;
                gs = from_bits(ab) / 2688.0f;
            }
            if (!(gs >= 0x1p-64f && gs <= 0x1p64f)) continue;
            const float rgs = 1.0f / gs;
            const float top = 2688.0f * gs;
            for (uint32_t xb = 0; xb < 0x7F81u; ++xb) {                /* every non-negative bf16 value, Inf included */
                const float m = from_bits(xb << 16);
                if (m > 4.0f * top && xb != 0x7F80u) continue;
                check_block_scale(m, gs, rgs);
            }
            uint32_t tb;
            memcpy(&tb, &top, 4);
            for (int j = 0; j < 4096; ++j) {
                uint32_t xb = (uint32_t)(rnd() % ((uint64_t)tb + 1u));
                if (j & 1) { xb = tb - (uint32_t)(rnd() % (1u << (j % 27))); if (xb > tb) xb = tb; }
                check_block_scale(from_bits(xb), gs, rgs);
            }
        }
        printf("checked %ld mismatches %ld\n", checked, bad);
        return bad == 0 ? 0 : 1;
    }
    if (mode == 4) {
        const float ds[3] = {6.0f, 448.0f, 2688.0f};
        uint32_t lo;
        const float lowest = 0x1p-100f;
        memcpy(&lo, &lowest, 4);
        for (int k = 0; k < 3; ++k) {
            const float d = ds[k], r = 1.0f / d;
            for (uint32_t u = lo; u < 0x7F800000u; ++u) {
                const float m = from_bits(u), want = m / d, q0 = m * r;
                const float got = fmaf(fmaf(-q0, d, m), r, q0);
                if (memcmp(&got, &want, 4) != 0) ++bad;
                ++checked;
            }
        }
        printf("checked %ld mismatches %ld\n", checked, bad);
        return bad == 0 ? 0 : 1;
    }
    if (mode == 2) {
        for (long it = 0; it < scales; ++it) {
            const float s = from_bits((uint32_t)(rnd() % 0x7F800000u));        /* +0 ... just below +Inf */
            for (int j = 0; j < 2048; ++j) {
                /* dividends around the scale (quotients of E4M3 size) and anywhere else */
                const uint32_t sb = (uint32_t)(rnd() % 0x7F800000u);
                const float x = (j & 1) ? from_bits(sb) : s * (float)((double)(rnd() % 100000) / 128.0);
                const float want = x / s, got = quotient_guarded(x, s);
                if (fabsf(want) < 0x1p-11f) {
                    if (!(fabsf(got) < 0x1p-10f)) ++bad;
                } else if (memcmp(&got, &want, 4) != 0 && !(isnan(got) && isnan(want))) {
                    ++bad;
                }
                ++checked;
            }
        }
        printf("checked %ld mismatches %ld\n", checked, bad);
        return bad == 0 ? 0 : 1;
    }
    for (long it = 0; it < scales; ++it) {
        uint32_t ab = (uint32_t)(rnd() % 0x7F000000u);
        if (mode == 0 && (it & 1)) ab &= 0xFFFF0000u;      /* a bf16 amax every other time */
        const float amax = from_bits(ab);
        float s = amax / 448.0f;
        if (s < 1e-12f) s = 1e-12f;
        if (!(s < 3.0e38f)) continue;
        const float y = 1.0f / s;
        if (mode == 0) {
            for (uint32_t xb = 0; xb < 0x8000u; ++xb) {   /* positive bf16 values order like their bits */
                const float x = from_bits(xb << 16);
                if (!(x <= amax)) break;
                check(x, s, y);
                check(-x, s, y);
            }
        } else {
            for (int j = 0; j < 4096; ++j) {
                uint32_t xb = (uint32_t)(rnd() % ((uint64_t)ab + 1u));
                if (j & 1) { xb = ab - (uint32_t)(rnd() % (1u << (j % 26))); if (xb > ab) xb = ab; }   /* near amax */
                check(from_bits(xb), s, y);
                check(-from_bits(xb), s, y);
            }
        }
    }
    printf("checked %ld mismatches %ld\n", checked, bad);
    return bad == 0 ? 0 : 1;
}
