// Host-only check (no GPU): the restatement's E4M3 encoder against the conversion routine
// that cuda_fp8.h provides for host code - the one `__nv_fp8_e4m3(float)` resolves to on
// the host.  TEST INFRASTRUCTURE ONLY.  Exit code 0 = identical on every probed input.
#include <cuda_fp8.h>
#include <cstdio>
#include <cstdint>
#include <cstring>
extern "C" {
#include "ref_restatement.c"
}
int main() {
    long bad = 0, n = 0;
    // every fp32 whose low 12 mantissa bits are one of a few patterns, over all exponents
    // and signs: covers every rounding boundary of the 3-bit mantissa, subnormals, overflow.
    const uint32_t lows[] = {0x000, 0x001, 0x7FF, 0x800, 0x801, 0xFFF};
    for (uint32_t hi = 0; hi < (1u << 20); hi++)
        for (uint32_t lo : lows) {
            uint32_t b = (hi << 12) | lo;
            float x; memcpy(&x, &b, 4);
            uint8_t want = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
            uint8_t got = rs_e4m3_from_float(x);
            bool nan = (b & 0x7FFFFFFFu) > 0x7F800000u;
            if (nan ? ((got & 0x7F) != 0x7F || (want & 0x7F) != 0x7F) : (got != want)) {
                if (bad < 10) printf("x=%a bits=%08x want=%02x got=%02x\n", x, b, want, got);
                bad++;
            }
            n++;
        }
    printf("checked %ld inputs, %ld mismatches\n", n, bad);
    return bad ? 1 : 0;
}
