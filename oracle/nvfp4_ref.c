/* CPU restatement of the reference's NVFP4 block quantiser, in plain C. TEST INFRASTRUCTURE ONLY:
 * the checker the CUDA quantiser is compared with, never a product path.
 *
 * Follows (paths inside the reference project):
 *   phasorkv/kernels/nvfp4.py:43-55   quantize_nv_block (block 16, E4M3 scale, fp32 tensor scale)
 *   phasorkv/quant.py:70-78           round_to: midpoints counted strictly below |y| => ties go DOWN
 *   phasorkv/quant.py:81-89           cast_e4m3: clamp to [0,448], round to nearest even
 *   phasorkv/kernels/nvfp4.py:21-36   code = magnitude index | sign<<3 (no signed zero), low nibble first
 * The E4M3 conversion is written out bit by bit so that it does not depend on any library cast.
 * Pinned against vectors produced by the reference (tests/golden/nvfp4_cases.npz).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float e4m3_to_float(uint8_t b) {
    int e = (b >> 3) & 15, m = b & 7;
    float v = e ? ldexpf(1.0f + m / 8.0f, e - 7) : ldexpf((float)m, -9);
    return (b & 0x80) ? -v : v;
}

/* non-negative finite x, already clamped to [0, 448] -> E4M3 byte, round to nearest even */
static uint8_t float_to_e4m3_rne(float x) {
    if (!(x > 0.0f)) return 0;
    int e;
    float fr = frexpf(x, &e);                 /* x = fr * 2^e, fr in [0.5, 1) */
    int E = e - 1;                            /* x = (2 fr) * 2^E, 2 fr in [1, 2) */
    if (E < -6) {                             /* subnormal: units of 2^-9 */
        float q = ldexpf(x, 9);
        float r = nearbyintf(q);              /* default rounding mode: nearest even */
        int m = (int)r;
        return (uint8_t)(m >= 8 ? 0x08 : m);  /* 8 * 2^-9 = 2^-6 is the first normal */
    }
    float q = ldexpf(fr, 4);                  /* (2 fr) * 8 in [8, 16) */
    int m = (int)nearbyintf(q);
    if (m == 16) { m = 8; E += 1; }
    if (E > 8 || (E == 8 && m > 14)) return 0x7E;      /* 448 = 1.75 * 2^8 is the largest finite */
    return (uint8_t)(((E + 7) << 3) | (m - 8));
}

static const float MID[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
static const float LEVEL[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* x [rows, width] fp32 (width % 16 == 0) -> codes [rows, width] (one code per byte),
 * scales [rows, width/16] E4M3 bytes, xhat [rows, width] (may be NULL). */
static void quantize_impl(const float* x, long rows, long width, float second, int scale_up,
                          uint8_t* codes, uint8_t* scales, float* xhat) {
    long nb = width / 16;
    for (long r = 0; r < rows; ++r)
        for (long b = 0; b < nb; ++b) {
            const float* xb = x + r * width + b * 16;
            float amax = 0.0f;
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(xb[i]));
            volatile float t0 = amax / 6.0f;      /* two divisions, in this order, each rounded to fp32 */
            volatile float t1 = t0 / second;
            float t = t1;
            if (t < 0.0f) t = 0.0f;
            if (t > 448.0f) t = 448.0f;
            uint8_t sb = float_to_e4m3_rne(t);
            /* quant.py:85-88 (PHASORKV_SCALE_UP=1): a scale rounded below the unclamped ratio moves one E4M3
             * step up; consecutive non-negative E4M3 values are consecutive bytes, 0x7e = 448 is the largest */
            if (scale_up && e4m3_to_float(sb) < t1 && sb < 0x7e) sb++;
            volatile float scale = e4m3_to_float(sb) * second;
            scales[r * nb + b] = sb;
            float div = scale < 1e-30f ? 1e-30f : scale;
            for (int i = 0; i < 16; ++i) {
                uint8_t code = 0;
                float v = 0.0f;
                if (scale > 0.0f) {
                    volatile float y = xb[i] / div;
                    float a = fabsf(y);
                    int idx = 0;
                    for (int k = 0; k < 7; ++k) idx += a > MID[k];
                    code = (uint8_t)(idx | ((idx > 0 && y < 0.0f) ? 8 : 0));
                    v = (y < 0.0f ? -LEVEL[idx] : LEVEL[idx]);
                }
                codes[r * width + b * 16 + i] = code;
                if (xhat) { volatile float p = v * scale; xhat[r * width + b * 16 + i] = p; }
            }
        }
}

void pkv_ref_nvfp4_quantize(const float* x, long rows, long width, float second,
                            uint8_t* codes, uint8_t* scales, float* xhat) {
    quantize_impl(x, rows, width, second, 0, codes, scales, xhat);
}

void pkv_ref_nvfp4_quantize_scale_up(const float* x, long rows, long width, float second,
                                     uint8_t* codes, uint8_t* scales, float* xhat) {
    quantize_impl(x, rows, width, second, 1, codes, scales, xhat);
}

/* inverse: value(code) * (scale * second) */
void pkv_ref_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, long rows, long width,
                              float second, float* out) {
    long nb = width / 16;
    for (long r = 0; r < rows; ++r)
        for (long b = 0; b < nb; ++b) {
            volatile float scale = e4m3_to_float(scales[r * nb + b]) * second;
            for (int i = 0; i < 16; ++i) {
                uint8_t c = codes[r * width + b * 16 + i];
                float v = LEVEL[c & 7];
                volatile float p = ((c & 8) ? -v : v) * scale;
                out[r * width + b * 16 + i] = p;
            }
        }
}

/* two codes per byte, even column in the low nibble */
void pkv_ref_pack_nibbles(const uint8_t* codes, long n, uint8_t* packed) {
    for (long i = 0; i < n / 2; ++i) packed[i] = (uint8_t)(codes[2 * i] | (codes[2 * i + 1] << 4));
}
