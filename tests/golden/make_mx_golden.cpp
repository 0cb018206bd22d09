// Regenerates the inputs of the reference's MXFP8 fixture and its CPU expectation, as a golden
// vector for the MXFP8 oracle (oracle/dk_oracle.py: mx_quant, mx_gemm_ref).
//
// The fixture (tests/unit/cdna4/warp/register/tile/mma_scaled.cu:206-258 of the reference, the same
// procedure as kernels/cdna4/gemm/mxfp8/MXFP8_8wave/8_wave_NT.cu:286-327): std::mt19937(123),
// std::normal_distribution<float>(0, 0.5), A [256,256] drawn first, then B [256,256]; per 1x32
// block e8m0 = clamp(floor(log2(amax)) + 127, 0, 254) (0 for an all-zero block),
// q = e4m3(x * 2^(127 - e8m0)); expectation c[i][j] = sum over blocks of
// (a_q * 2^(sa-127)) * (b_q * 2^(sb-127)) accumulated in fp32 in k order.
// This file restates that procedure step by step (test infrastructure; the e8m0 rule is the
// fixture's own formula); the float -> e4m3 conversion is this repository's own (round to nearest
// even, saturating at 448).
//
// Output (binary, little endian) on stdout: the first ROWS rows of A and of B as fp32, their e4m3
// bytes and e8m0 scales, and c_ref [ROWS, ROWS]. make_golden.py turns it into mx_fixture.npz.
//   g++ -O2 -o make_mx_golden make_mx_golden.cpp && ./make_mx_golden > mx_fixture.bin
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

static uint8_t f32_to_e4m3(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    float a = std::fabs(x);
    if (std::isnan(a)) return (uint8_t)(sign | 0x7f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (a < 0.0009765625f) return sign;
    int e;
    (void)std::frexp(a, &e);
    int exp = std::max(e - 1, -6);
    const float ulp = std::ldexp(1.0f, exp - 3);
    float v = std::nearbyint(a / ulp) * ulp;
    if (v >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (v == 0.0f) return sign;
    int e2;
    (void)std::frexp(v, &e2);
    int ex = e2 - 1;
    if (ex < -6) return (uint8_t)(sign | (uint8_t)(int)(v / std::ldexp(1.0f, -9)));
    const int man = (int)(v / std::ldexp(1.0f, ex - 3)) - 8;
    return (uint8_t)(sign | (uint8_t)((ex + 7) << 3) | (uint8_t)man);
}
static float e4m3_to_f32(uint8_t b) {
    const int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v = e == 0 ? std::ldexp((float)m, -9) : std::ldexp(1.0f + m / 8.0f, e - 7);
    return s ? -v : v;
}
static uint8_t e8m0_of(const float* v, int n) {
    float mx = 0.f;
    for (int i = 0; i < n; ++i) mx = std::max(mx, std::fabs(v[i]));
    if (mx == 0.f) return 0;
    return (uint8_t)std::clamp((int)std::floor(std::log2(mx)) + 127, 0, 254);
}

int main() {
    constexpr int M = 256, N = 256, K = 256, SK = K / 32, ROWS = 64;
    std::mt19937 rng(123);
    std::normal_distribution<float> dist(0.0f, 0.5f);
    std::vector<float> a(M * K), b(N * K);
    for (auto& v : a) v = dist(rng);
    for (auto& v : b) v = dist(rng);
    std::vector<uint8_t> aq(M * K), bq(N * K), sa(M * SK), sb(N * SK);
    auto quant = [&](const std::vector<float>& src, std::vector<uint8_t>& q, std::vector<uint8_t>& s, int rows) {
        for (int r = 0; r < rows; ++r)
            for (int kb = 0; kb < SK; ++kb) {
                const float* blk = &src[r * K + kb * 32];
                const uint8_t e = e8m0_of(blk, 32);
                s[r * SK + kb] = e;
                const float inv = std::ldexp(1.0f, 127 - (int)e);
                for (int i = 0; i < 32; ++i) q[r * K + kb * 32 + i] = f32_to_e4m3(blk[i] * inv);
            }
    };
    quant(a, aq, sa, M);
    quant(b, bq, sb, N);
    std::vector<float> c(ROWS * ROWS);
    for (int i = 0; i < ROWS; ++i)
        for (int j = 0; j < ROWS; ++j) {
            float acc = 0.f;
            for (int kb = 0; kb < SK; ++kb) {
                const float fa = std::ldexp(1.0f, (int)sa[i * SK + kb] - 127);
                const float fb = std::ldexp(1.0f, (int)sb[j * SK + kb] - 127);
                for (int ki = 0; ki < 32; ++ki)
                    acc += e4m3_to_f32(aq[i * K + kb * 32 + ki]) * fa * e4m3_to_f32(bq[j * K + kb * 32 + ki]) * fb;
            }
            c[i * ROWS + j] = acc;
        }
    std::fwrite(a.data(), 4, ROWS * K, stdout);
    std::fwrite(b.data(), 4, ROWS * K, stdout);
    std::fwrite(aq.data(), 1, ROWS * K, stdout);
    std::fwrite(bq.data(), 1, ROWS * K, stdout);
    std::fwrite(sa.data(), 1, ROWS * SK, stdout);
    std::fwrite(sb.data(), 1, ROWS * SK, stdout);
    std::fwrite(c.data(), 4, ROWS * ROWS, stdout);
    return 0;
}
