/* Plain-C restatement of the integer/byte parts of the hot path. TEST INFRASTRUCTURE ONLY: loaded by
 * tests and by the benchmark's CPU-baseline leg, never by the product.
 *
 *   oracle_moe_align          - prime_moe/csrc/kernels/fused_moe_bf16_kernel.cu:853-907 (histogram,
 *                               padded scan, -1 fill, expert_ids by binary search, scatter); the order
 *                               inside an expert, which the reference leaves to atomics, is ascending
 *   oracle_pack_scales_blocked- prime_moe/__init__.py:106-115 (byte permutation into 512-byte tiles)
 *   oracle_mx_quantize        - test/test_mxfp8.py:21-38 (shared exponent = fp32 exponent field - 8,
 *                               clamp [0,254]; values scaled by 2^(127-e), saturated to +-448, rounded
 *                               to e4m3 nearest-even)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

int oracle_moe_align(const int32_t *ids, int n, int num_experts, int block_m, int pad_to, int max_padded,
                     int max_blocks, int32_t *sorted, int32_t *expert_ids, int32_t *npp) {
    int *offs = (int *)calloc((size_t)num_experts + 1, sizeof(int));
    int *fill = (int *)calloc((size_t)num_experts, sizeof(int));
    if (!offs || !fill) return 1;
    for (int i = 0; i < n; ++i)
        if (ids[i] >= 0 && ids[i] < num_experts) offs[ids[i] + 1] += 1;
    for (int e = 0; e < num_experts; ++e) {
        int padded = (offs[e + 1] + pad_to - 1) / pad_to * pad_to;
        offs[e + 1] = offs[e] + padded;
    }
    const int total = offs[num_experts];
    *npp = total;
    for (int i = 0; i < max_padded; ++i) sorted[i] = -1;
    for (int j = 0; j < max_blocks; ++j) {
        const int row = j * block_m;
        if (row >= total) {
            expert_ids[j] = num_experts - 1;
            continue;
        }
        int lo = 0, hi = num_experts - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (offs[mid] <= row) lo = mid;
            else hi = mid - 1;
        }
        expert_ids[j] = lo;
    }
    for (int i = 0; i < n; ++i) {
        const int e = ids[i];
        if (e < 0 || e >= num_experts) continue;
        sorted[offs[e] + fill[e]++] = i;
    }
    free(offs);
    free(fill);
    return 0;
}

/* scales: [lead][mn][kb] bytes -> out: [lead][mn*kb] bytes */
void oracle_pack_scales_blocked(const uint8_t *scales, uint8_t *out, long lead, int mn, int kb) {
    for (long l = 0; l < lead; ++l) {
        const uint8_t *src = scales + l * (long)mn * kb;
        uint8_t *dst = out + l * (long)mn * kb;
        for (int r = 0; r < mn; ++r)
            for (int k = 0; k < kb; ++k) {
                long tile = (long)(r / 128) * (kb / 4) + k / 4;
                dst[tile * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + k % 4] = src[(long)r * kb + k];
            }
    }
}

/* round-to-nearest-even conversion of a float (|v| <= 448 after clamping) to e4m3fn bits */
static uint8_t float_to_e4m3(float v) {
    uint8_t sign = v < 0 || (v == 0 && signbit(v)) ? 0x80 : 0;
    float a = fabsf(v);
    if (isnan(a)) return sign | 0x7f;
    if (a > 448.f) a = 448.f;
    if (a == 0.f) return sign;
    int ex;
    frexpf(a, &ex);          /* a = m * 2^ex, m in [0.5, 1) -> unbiased exponent ex-1 */
    int e = ex - 1;
    if (e < -6) e = -6;      /* subnormal range: quantum 2^-9 */
    float quantum = ldexpf(1.f, e - 3);
    float q = nearbyintf(a / quantum);   /* ties-to-even in the default rounding mode */
    float r = q * quantum;
    if (r > 448.f) r = 448.f;
    if (r == 0.f) return sign;
    frexpf(r, &ex);
    e = ex - 1;
    if (e < -6) {            /* subnormal */
        int mant = (int)(r / ldexpf(1.f, -9));
        return sign | (uint8_t)mant;
    }
    int mant = (int)((r / ldexpf(1.f, e) - 1.f) * 8.f);
    return sign | (uint8_t)(((e + 7) << 3) | mant);
}

/* t: [rows][k] floats -> q: [rows][k] e4m3 bytes, scales: [rows][k/32] e8m0 bytes */
void oracle_mx_quantize(const float *t, long rows, int k, uint8_t *q, uint8_t *scales) {
    const int nb = k / 32;
    for (long r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const float *g = t + r * (long)k + b * 32;
            float amax = 0.f;
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(g[i]));
            uint32_t bits;
            memcpy(&bits, &amax, 4);
            int e = (int)((bits >> 23) & 0xff) - 8;
            if (e < 0) e = 0;
            if (e > 254) e = 254;
            scales[r * (long)nb + b] = (uint8_t)e;
            const float inv = ldexpf(1.f, 127 - e);
            for (int i = 0; i < 32; ++i) {
                float v = g[i] * inv;
                if (v > 448.f) v = 448.f;
                if (v < -448.f) v = -448.f;
                q[r * (long)k + b * 32 + i] = float_to_e4m3(v);
            }
        }
}
