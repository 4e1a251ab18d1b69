// ternarise.cpp -- real-valued weights -> {-1, 0, +1} with one scale per matrix (host C++).
//
// The reference only generates synthetic ternary matrices (main.cu:248-265); a model's weights
// have to be made ternary before they can be encoded.  This is the absmean rule of BitNet b1.58:
//     scale = mean(|W|) over the whole matrix
//     W_t   = clamp(round_half_even(W / (scale + 1e-5)), -1, +1)
// so that W ~ scale * W_t.  The mean is a double-precision sum taken column by column and added in
// column order (the same result whatever the number of threads); everything else is fp32.
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "internal.h"

using namespace sptmm;

static float half_to_float(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {                                   // subnormal: renormalise
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline float element(const void *W, uint32_t dtype, size_t i)
{
    return dtype == SPTMM_F16 ? half_to_float(static_cast<const uint16_t *>(W)[i]) : static_cast<const float *>(W)[i];
}

extern "C" int sptmm_ternarise_absmean(const void *W, uint32_t dtype, uint32_t K, uint32_t N, int8_t *W_ternary, float *scale)
{
    if (!W || !W_ternary) return fail(SPTMM_ERR_INVALID, "ternarise_absmean: null pointer");
    if (dtype != SPTMM_F16 && dtype != SPTMM_F32) return fail(SPTMM_ERR_INVALID, "ternarise_absmean: weights must be fp16 or fp32");
    if (K == 0 || N == 0) return fail(SPTMM_ERR_INVALID, "ternarise_absmean: K=%u N=%u", K, N);
    const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    const unsigned nt = std::min<unsigned>(hw, N);
    std::vector<double> colsum(N, 0.0);
    auto over_columns = [&](auto &&body) {
        std::vector<std::thread> th;
        for (unsigned t = 0; t < nt; t++)
            th.emplace_back([&, t] { for (uint32_t c = t; c < N; c += nt) body(c); });
        for (auto &x : th) x.join();
    };
    over_columns([&](uint32_t c) {
        double s = 0.0;
        for (uint32_t k = 0; k < K; k++) s += std::fabs((double)element(W, dtype, (size_t)c * K + k));
        colsum[c] = s;
    });
    double total = 0.0;
    for (uint32_t c = 0; c < N; c++) total += colsum[c];
    const float mean = (float)(total / ((double)K * N));
    if (!std::isfinite(mean)) return fail(SPTMM_ERR_INVALID, "ternarise_absmean: the matrix holds a NaN or an infinity");
    const float inv = 1.0f / (mean + 1e-5f);
    over_columns([&](uint32_t c) {
        for (uint32_t k = 0; k < K; k++) {
            const float q = nearbyintf(element(W, dtype, (size_t)c * K + k) * inv);      // round half to even
            W_ternary[(size_t)c * K + k] = (int8_t)(q > 1.0f ? 1 : (q < -1.0f ? -1 : (int)q));
        }
    });
    if (scale) *scale = mean;
    return SPTMM_OK;
}
