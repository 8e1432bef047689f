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
 * usage: quotient_check <scales> <mode>    mode 0: every bf16 dividend up to amax; mode 1: random fp32 dividends;
 *                                          mode 2: given scales of any size, random dividends
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

static long checked = 0, bad = 0;
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
