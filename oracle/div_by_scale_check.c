/* Test infrastructure (CPU only; nothing in the product path uses this file).
 *
 * The u8 KV quantiser divides every value of a row by the row's scale, q = RN(x / s), and its result has to be
 * reproducible bit for bit.  The GPU store kernel for 16-bit rows replaces the IEEE division by
 *     r = RN(1 / s);  q0 = RN(x * r);  e = fma(-s, q0, x);  q = fma(e, r, q0)
 * and falls back to the division itself for |x| < 1e-30.  This program checks, for EVERY positive finite f16-valued
 * scale (the scale is stored as f16) and EVERY f16- and bf16-valued x, that the two agree.  Exit code 0 = they do.
 *
 *     gcc -O2 -mfma -o div_by_scale_check div_by_scale_check.c -lm && ./div_by_scale_check [stride]
 *
 * `stride` > 1 visits every stride-th scale (a quick run for the test suite); 1 is the exhaustive run (4.2e9 pairs,
 * about half a minute).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static float half_bits_to_float(uint16_t h) {
    uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023, u;
    if (e == 0) {
        if (m == 0) {
            u = s << 31;
        } else {
            int k = 0;
            while (!(m & 1024)) {
                m <<= 1;
                ++k;
            }
            m &= 1023;
            u = (s << 31) | ((uint32_t)(127 - 15 - k + 1) << 23) | (m << 13);
        }
    } else if (e == 31) {
        u = (s << 31) | 0x7f800000u | (m << 13);
    } else {
        u = (s << 31) | ((e - 15 + 127) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static float bfloat_bits_to_float(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

int main(int argc, char** argv) {
    const uint32_t stride = argc > 1 ? (uint32_t)atoi(argv[1]) : 1;
    unsigned long long bad = 0, n = 0;
    for (uint32_t hs = 1; hs < 0x7c00; hs += stride ? stride : 1) {
        const float s = half_bits_to_float((uint16_t)hs), r = 1.0f / s;
        for (uint32_t xi = 0; xi < 131072; ++xi) {
            const float x = xi < 65536 ? half_bits_to_float((uint16_t)xi) : bfloat_bits_to_float((uint16_t)(xi - 65536));
            const float want = x / s;
            float got;
            if (fabsf(x) < 1e-30f) {
                got = x / s;
            } else {
                const float q0 = x * r;
                got = isfinite(q0) ? fmaf(fmaf(-s, q0, x), r, q0) : q0;
            }
            ++n;
            if (!(want == got || (isnan(want) && isnan(got)))) {
                if (bad < 10) printf("mismatch s=%a x=%a division=%a fma form=%a\n", s, x, want, got);
                ++bad;
            }
        }
    }
    printf("checked %llu pairs, %llu mismatches\n", n, bad);
    return bad != 0;
}
