/*
 * Plain-C restatement of the integer / byte part of the MoE path: routing, permutation,
 * 128x128 block quantisation to e4m3. TEST INFRASTRUCTURE ONLY: linked by tests/ (and usable as
 * a CPU baseline), never by the product path.
 *
 * The reference has no MoE code; the definitions are those of oracle/dk_oracle.py, whose block
 * quantiser follows the pattern of the reference's block-scaled fixtures
 * (tests/unit/cdna4/warp/register/tile/mma_scaled.cu:200-258) with 128x128 fp32 scale blocks.
 * Parity of these functions is UNPINNED by the reference; this file and the Python oracle pin each
 * other (tests/test_oracle_cpu.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* top-k on raw fp32 logits, ties to the lower expert index, slots in descending logit order;
 * weights = softmax over all experts, gathered and renormalised. */
void dk_c_route(const float* logits, int T, int E, int k, int32_t* idx, float* w) {
    uint8_t* taken = (uint8_t*)malloc((size_t)E);
    for (int t = 0; t < T; ++t) {
        const float* row = logits + (size_t)t * E;
        memset(taken, 0, (size_t)E);
        float m = -INFINITY;
        for (int e = 0; e < E; ++e) m = row[e] > m ? row[e] : m;
        float denom = 0.f;
        for (int e = 0; e < E; ++e) denom += expf(row[e] - m);
        float sum = 0.f;
        for (int j = 0; j < k; ++j) {
            int best = -1;
            for (int e = 0; e < E; ++e)
                if (!taken[e] && (best < 0 || row[e] > row[best])) best = e;
            taken[best] = 1;
            idx[(size_t)t * k + j] = best;
            w[(size_t)t * k + j] = expf(row[best] - m) / denom;
            sum += w[(size_t)t * k + j];
        }
        for (int j = 0; j < k; ++j) w[(size_t)t * k + j] /= sum;
    }
    free(taken);
}

/* stable counting sort of the T*k pairs by expert; experts cut into segments of `seg`, row
 * numbering restarts per segment, every expert padded to `pad` rows.
 * offsets: [E/seg][seg+1]; pair_of_row: [E/seg][cap], -1 on padding rows. */
void dk_c_permute(const int32_t* idx, int T, int k, int E, int pad, int seg, int cap,
                  int32_t* row_of_pair, int32_t* pair_of_row, int32_t* offsets, int32_t* counts) {
    const int n = T * k, nseg = E / seg;
    memset(counts, 0, sizeof(int32_t) * (size_t)E);
    for (int i = 0; i < n; ++i) counts[idx[i]]++;
    for (int g = 0; g < nseg; ++g) {
        int run = 0;
        for (int j = 0; j < seg; ++j) {
            offsets[g * (seg + 1) + j] = run;
            run += (counts[g * seg + j] + pad - 1) / pad * pad;
        }
        offsets[g * (seg + 1) + seg] = run;
    }
    for (size_t i = 0; i < (size_t)nseg * cap; ++i) pair_of_row[i] = -1;
    int32_t* fill = (int32_t*)calloc((size_t)E, sizeof(int32_t));
    for (int i = 0; i < n; ++i) {            /* (token, slot) order */
        const int e = idx[i], g = e / seg;
        const int row = offsets[g * (seg + 1) + (e - g * seg)] + fill[e]++;
        row_of_pair[i] = row;
        pair_of_row[(size_t)g * cap + row] = i;
    }
    free(fill);
}

static float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* float -> e4m3 (fn: no infinities, max 448), round to nearest even, saturating */
static uint8_t f32_to_e4m3(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    float a = fabsf(x);
    if (isnan(a)) return (uint8_t)(sign | 0x7f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (a < 0.0009765625f) return sign;                 /* below half the smallest subnormal (2^-10) */
    int e;
    (void)frexpf(a, &e);                                /* a = m * 2^e, m in [0.5, 1) */
    int exp = e - 1;                                    /* a = 1.xxx * 2^exp */
    if (exp < -6) exp = -6;                             /* subnormal range: spacing 2^-9 */
    const float ulp = ldexpf(1.0f, exp - 3);            /* 3 mantissa bits */
    float q = a / ulp;                                  /* exact: power-of-two scaling */
    float r = nearbyintf(q);                            /* default rounding mode: nearest even */
    float v = r * ulp;
    if (v >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (v == 0.0f) return sign;
    int e2;
    (void)frexpf(v, &e2);
    int ex = e2 - 1;
    if (ex < -6) {                                      /* subnormal */
        const int man = (int)(v / ldexpf(1.0f, -9));
        return (uint8_t)(sign | (uint8_t)man);
    }
    const int man = (int)(v / ldexpf(1.0f, ex - 3)) - 8;
    return (uint8_t)(sign | (uint8_t)((ex + 7) << 3) | (uint8_t)man);
}

/* x: bf16 bits [R, C]; q: [R, C] bytes; s: [R/128, C/128] */
void dk_c_quant_block128(const uint16_t* x, int R, int C, uint8_t* q, float* s) {
    for (int br = 0; br < R / 128; ++br)
        for (int bc = 0; bc < C / 128; ++bc) {
            float amax = 0.f;
            for (int r = 0; r < 128; ++r)
                for (int c = 0; c < 128; ++c) {
                    const float v = fabsf(bf16_to_f32(x[(size_t)(br * 128 + r) * C + bc * 128 + c]));
                    amax = v > amax ? v : amax;
                }
            const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
            s[(size_t)br * (C / 128) + bc] = scale;
            for (int r = 0; r < 128; ++r)
                for (int c = 0; c < 128; ++c) {
                    const size_t i = (size_t)(br * 128 + r) * C + bc * 128 + c;
                    float y = bf16_to_f32(x[i]) / scale;
                    y = y > 448.0f ? 448.0f : (y < -448.0f ? -448.0f : y);
                    q[i] = f32_to_e4m3(y);
                }
        }
}
