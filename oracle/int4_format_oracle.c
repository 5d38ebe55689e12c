/*
 * int4_format_oracle.c - CPU restatement of the reference's weight-only INT4 format.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing that ships (the CUDA library, its host code, the
 * Python wrapper) may link, load or call this file. It exists so the parity tests and the
 * bench's CPU baseline have an independent statement of the format to check the GPU path
 * against. Parity is PINNED: tests/test_oracle_format.py checks this file against every
 * known-answer vector of the reference's own format gate (tests/quantization_format_test.c)
 * and, where the reference sources are present, bit-for-bit against the reference's
 * csrc/linear_weight.cpp compiled as oracle/_ref/libref_linear_weight.so.
 *
 * The format (reference: csrc/include/linear_weight.h:46-54, csrc/linear_weight.cpp):
 *   - symmetric signed 4-bit codes in [-7, 7]; the nibble 0x8 (-8) is reserved and invalid
 *   - one BF16 scale per 128 consecutive K elements of a row
 *   - scale = BF16_RNE(max|w| / 7) over the group, 1.0 for an all-zero group
 *   - code  = clip(round_half_even(w / scale_rounded), -7, 7)
 *   - byte j of a row holds K index 2j in its low nibble and 2j+1 in its high nibble
 *   - dequantized weight = (float)code * (float)scale, an exact FP32 product
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORC_GROUP 128
#define ORC_TILE_ROWS 8
#define ORC_QMAX 7

enum {
    ORC_OK = 0,
    ORC_ERR_ARG = 1,    /* null pointer */
    ORC_ERR_RANGE = 2,  /* extent the format cannot hold */
    ORC_ERR_VALUE = 3,  /* non-finite weight, or a scale that rounds to <= 0 / non-finite */
    ORC_ERR_FORMAT = 4, /* reserved code or bad scale met while reading */
};

/* FP32 -> BF16, round to nearest even on the discarded 16 bits.
 * Follows linear_f32_to_bf16 (csrc/linear_weight.cpp:34-44). */
uint16_t orc_f32_to_bf16(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* BF16 -> FP32 widening. Follows linear_bf16_to_f32 (csrc/linear_weight.cpp:46-51). */
float orc_bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float v;
    memcpy(&v, &u, 4);
    return v;
}

/* Extent rules of linear_layout_init (csrc/linear_weight.cpp:57-86): positive extents,
 * group exactly 128, K a whole number of groups, N a whole number of 8-row tiles. */
int orc_layout(long long n, long long k, long long group, long long *packed_bytes,
               long long *scale_count) {
    if (!packed_bytes || !scale_count) return ORC_ERR_ARG;
    if (n <= 0 || k <= 0) return ORC_ERR_RANGE;
    if (group != ORC_GROUP) return ORC_ERR_RANGE;
    if (k % group) return ORC_ERR_RANGE;
    if (n % ORC_TILE_ROWS) return ORC_ERR_RANGE;
    *packed_bytes = n * k / 2;
    *scale_count = n * (k / group);
    return ORC_OK;
}

static int nibble_to_code(int nib) { return nib & 8 ? nib - 16 : nib; }

/* Sign-extended code at (row, k). Follows linear_packed_code (csrc/linear_weight.cpp:96-102). */
int orc_packed_code(const uint8_t *packed, long long row, long long k, long long k_extent) {
    const uint8_t b = packed[(row * k_extent + k) >> 1];
    return nibble_to_code((k & 1) ? (b >> 4) : (b & 15));
}

/* Quantize FP32 [n, k] row-major. Follows linear_quantize_int4 (csrc/linear_weight.cpp:108-176):
 * all inputs are validated before any output byte is written. */
int orc_quantize(long long n, long long k, const float *w, uint8_t *packed, uint16_t *scales) {
    long long pb, sc;
    if (!w || !packed || !scales) return ORC_ERR_ARG;
    const int st = orc_layout(n, k, ORC_GROUP, &pb, &sc);
    if (st) return st;
    for (long long i = 0; i < n * k; ++i)
        if (!isfinite(w[i])) return ORC_ERR_VALUE;
    const long long gpr = k / ORC_GROUP;
    /* scales first, so a refused scale leaves the payload untouched as the reference does */
    for (long long g = 0; g < n * gpr; ++g) {
        const float *src = w + g * ORC_GROUP;
        float m = 0.0f;
        for (int i = 0; i < ORC_GROUP; ++i) {
            const float a = fabsf(src[i]);
            if (a > m) m = a;
        }
        const uint16_t bits = orc_f32_to_bf16(m == 0.0f ? 1.0f : m / (float)ORC_QMAX);
        const float s = orc_bf16_to_f32(bits);
        if (!(s > 0.0f) || !isfinite(s)) return ORC_ERR_VALUE;
    }
    for (long long g = 0; g < n * gpr; ++g) {
        const float *src = w + g * ORC_GROUP;
        uint8_t *dst = packed + g * (ORC_GROUP / 2);
        float m = 0.0f;
        for (int i = 0; i < ORC_GROUP; ++i) {
            const float a = fabsf(src[i]);
            if (a > m) m = a;
        }
        const uint16_t bits = orc_f32_to_bf16(m == 0.0f ? 1.0f : m / (float)ORC_QMAX);
        const float s = orc_bf16_to_f32(bits);
        scales[g] = bits;
        for (int i = 0; i < ORC_GROUP; i += 2) {
            int c[2];
            for (int j = 0; j < 2; ++j) {
                float q = nearbyintf(src[i + j] / s); /* default rounding mode: half to even */
                if (q > (float)ORC_QMAX) q = (float)ORC_QMAX;
                if (q < -(float)ORC_QMAX) q = -(float)ORC_QMAX;
                c[j] = (int)q;
            }
            dst[i >> 1] = (uint8_t)((c[0] & 15) | ((c[1] & 15) << 4));
        }
    }
    return ORC_OK;
}

/* Dequantize to FP32 [n, k]. Follows linear_dequantize_int4 (csrc/linear_weight.cpp:178-216):
 * refuses the reserved nibble 0x8 and a scale that is not positive and finite. */
int orc_dequantize(long long n, long long k, const uint8_t *packed, const uint16_t *scales,
                   float *out) {
    long long pb, sc;
    if (!packed || !scales || !out) return ORC_ERR_ARG;
    const int st = orc_layout(n, k, ORC_GROUP, &pb, &sc);
    if (st) return st;
    const long long gpr = k / ORC_GROUP;
    for (long long g = 0; g < n * gpr; ++g) {
        const float s = orc_bf16_to_f32(scales[g]);
        if (!(s > 0.0f) || !isfinite(s)) return ORC_ERR_FORMAT;
        const uint8_t *src = packed + g * (ORC_GROUP / 2);
        float *dst = out + g * ORC_GROUP;
        for (int j = 0; j < ORC_GROUP / 2; ++j) {
            const int lo = src[j] & 15, hi = src[j] >> 4;
            if (lo == 8 || hi == 8) return ORC_ERR_FORMAT;
            dst[2 * j] = (float)nibble_to_code(lo) * s;
            dst[2 * j + 1] = (float)nibble_to_code(hi) * s;
        }
    }
    return ORC_OK;
}

/* ---- dense kernels used by the FFN oracle (plain C so the CPU baseline is not numpy-bound) ---- */

/* out[m, n] (FP64) = sum_k a[m, k] * w[n, k]; a and w are FP32, accumulation is FP64.
 * This is the "float64 matmul of the dequantized weight" the reference's kernel gate uses
 * (tests/test_quantization_kernel.py:115). */
void orc_matmul_f64(int m, long long n, long long k, const float *a, const float *w, double *out) {
    for (int i = 0; i < m; ++i) {
        for (long long r = 0; r < n; ++r) {
            const float *wr = w + r * k;
            const float *ar = a + (long long)i * k;
            double acc0 = 0.0, acc1 = 0.0, acc2 = 0.0, acc3 = 0.0;
            long long j = 0;
            for (; j + 3 < k; j += 4) {
                acc0 += (double)ar[j] * (double)wr[j];
                acc1 += (double)ar[j + 1] * (double)wr[j + 1];
                acc2 += (double)ar[j + 2] * (double)wr[j + 2];
                acc3 += (double)ar[j + 3] * (double)wr[j + 3];
            }
            for (; j < k; ++j) acc0 += (double)ar[j] * (double)wr[j];
            out[(long long)i * n + r] = (acc0 + acc1) + (acc2 + acc3);
        }
    }
}

/* The same product read straight from the packed payload (dequantize inside the loop), FP64
 * accumulation. Used for shapes whose FP32 dequantized copy would not fit comfortably. */
int orc_matmul_packed_f64(int m, long long n, long long k, const float *a, const uint8_t *packed,
                          const uint16_t *scales, double *out) {
    const long long gpr = k / ORC_GROUP;
    if (k % ORC_GROUP) return ORC_ERR_RANGE;
    for (long long r = 0; r < n; ++r) {
        for (int i = 0; i < m; ++i) out[(long long)i * n + r] = 0.0;
        for (long long g = 0; g < gpr; ++g) {
            const float s = orc_bf16_to_f32(scales[r * gpr + g]);
            const uint8_t *src = packed + (r * k + g * ORC_GROUP) / 2;
            float wv[ORC_GROUP];
            for (int j = 0; j < ORC_GROUP / 2; ++j) {
                wv[2 * j] = (float)nibble_to_code(src[j] & 15) * s;
                wv[2 * j + 1] = (float)nibble_to_code(src[j] >> 4) * s;
            }
            for (int i = 0; i < m; ++i) {
                const float *ar = a + (long long)i * k + g * ORC_GROUP;
                double acc = 0.0;
                for (int j = 0; j < ORC_GROUP; ++j) acc += (double)ar[j] * (double)wv[j];
                out[(long long)i * n + r] += acc;
            }
        }
    }
    return ORC_OK;
}
