// cli_encode.cpp -- offline encoder: bin/sptmm_encode writes an encoded-weights file.
//
//   sptmm_encode -K 6912 -N 2560 -S 4096 -format u16_v256 -o w.sptmm         reference generator
//   sptmm_encode -K 8192 -N 28672 -p0 0.5 -seed 7 -format delta_lane -o w.sptmm      i.i.d. entries
//   sptmm_encode -K 6912 -N 2560 -dense W.i8 -format u16_div -split 32 -S 4096 -o w.sptmm
//   sptmm_encode -K 6912 -N 2560 -f32 W.f32 -o w.sptmm      real weights, made ternary first (absmean)
//
// -dense names a raw file of K*N int8 values in {-1,0,+1}, column-major (column c at bytes
// c*K .. c*K+K-1), i.e. W_work as the reference holds it (main.cu:917).  -f32 / -f16 name a raw file
// of K*N real weights in the same order; they are made ternary with sptmm_ternarise_absmean and the
// scale is printed (the factor a de-quantising epilogue multiplies by).  No GPU is touched.
// The reference has no such tool: it regenerates and re-encodes on the GPU at every start.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/sptmm.h"

namespace {

[[noreturn]] void die(const std::string &msg)
{
    fprintf(stderr, "sptmm_encode: %s\n", msg.c_str());
    exit(EXIT_FAILURE);
}

uint32_t format_of(const std::string &s)
{
    if (s == "u16_v256") return SPTMM_FMT_U16_V256;
    if (s == "delta_lane") return SPTMM_FMT_DELTA_LANE;
    if (s == "u16_div") return SPTMM_FMT_U16_DIV;
    if (s == "delta_div256") return SPTMM_FMT_DELTA_DIV256;
    if (s == "i2s") return SPTMM_FMT_I2S;
    die("unknown -format '" + s + "' (u16_v256, delta_lane, u16_div, delta_div256, i2s)");
}

}  // namespace

int main(int argc, char **argv)
{
    uint64_t K = 0, N = 0, S = 0, split = 32, seed = 0;
    double p0 = -1.0;
    std::string format = "u16_v256", out, dense, real;
    uint32_t real_dtype = SPTMM_F32;
    for (int i = 1; i < argc; i++) {
        std::string key(argv[i]), val;
        while (!key.empty() && key[0] == '-') key.erase(0, 1);
        const size_t eq = key.find('=');
        if (eq != std::string::npos) { val = key.substr(eq + 1); key = key.substr(0, eq); }
        else if (i + 1 < argc) val = argv[++i];
        else die("flag -" + key + " needs a value");
        if (key == "K") K = strtoull(val.c_str(), nullptr, 10);
        else if (key == "N") N = strtoull(val.c_str(), nullptr, 10);
        else if (key == "S") S = strtoull(val.c_str(), nullptr, 10);
        else if (key == "split") split = strtoull(val.c_str(), nullptr, 10);
        else if (key == "seed") seed = strtoull(val.c_str(), nullptr, 10);
        else if (key == "p0") p0 = atof(val.c_str());
        else if (key == "format") format = val;
        else if (key == "o") out = val;
        else if (key == "dense") dense = val;
        else if (key == "f32") { real = val; real_dtype = SPTMM_F32; }
        else if (key == "f16") { real = val; real_dtype = SPTMM_F16; }
        else die("unknown flag -" + key);
    }
    if (K == 0 || N == 0 || out.empty()) die("usage: sptmm_encode -K k -N n (-S s | -p0 p [-seed x] | -dense file | -f32 file | -f16 file) [-format f] [-split s] -o file");
    if (K >= 65536 || N > (1u << 24)) die("K must be below 65536 and N at most 2^24");
    std::vector<int8_t> W(K * N);
    if (!real.empty()) {
        const size_t es = real_dtype == SPTMM_F16 ? 2 : 4;
        std::vector<unsigned char> raw(K * N * es);
        FILE *f = fopen(real.c_str(), "rb");
        if (!f) die("cannot open " + real);
        const size_t got = fread(raw.data(), 1, raw.size(), f);
        const bool more = fgetc(f) != EOF;
        fclose(f);
        if (got != raw.size() || more) die(real + " does not hold exactly K*N values");
        float scale = 0.0f;
        if (sptmm_ternarise_absmean(raw.data(), real_dtype, (uint32_t)K, (uint32_t)N, W.data(), &scale) != SPTMM_OK) die(sptmm_last_error());
        printf("absmean scale %.9g\n", scale);
    } else if (!dense.empty()) {
        FILE *f = fopen(dense.c_str(), "rb");
        if (!f) die("cannot open " + dense);
        const size_t got = fread(W.data(), 1, W.size(), f);
        const bool more = fgetc(f) != EOF;
        fclose(f);
        if (got != W.size() || more) die(dense + " does not hold exactly K*N bytes");
    } else if (p0 >= 0.0) {
        if (sptmm_gen_ternary_iid((uint32_t)K, (uint32_t)N, p0, seed, W.data()) != SPTMM_OK) die(sptmm_last_error());
    } else {
        if (S == 0) die("one of -S (reference generator), -p0 (i.i.d.) or -dense is needed");
        if (sptmm_gen_ternary_fixed((uint32_t)K, (uint32_t)N, (uint32_t)S, W.data()) != SPTMM_OK) die(sptmm_last_error());
    }
    const uint32_t fmt = format_of(format);
    const bool reference_layout = fmt == SPTMM_FMT_U16_DIV || fmt == SPTMM_FMT_DELTA_DIV256;
    sptmm_weights *w = nullptr;
    if (sptmm_encode(W.data(), (uint32_t)K, (uint32_t)N, fmt, (uint32_t)split, reference_layout ? (uint32_t)S : 0u, &w) != SPTMM_OK)
        die(sptmm_last_error());
    if (sptmm_weights_save(w, out.c_str()) != SPTMM_OK) die(sptmm_last_error());
    sptmm_weights_info info;
    sptmm_weights_info_get(w, &info);
    printf("%s: %s K=%u N=%u nnz=%llu stream_bytes=%llu\n", out.c_str(), format.c_str(), info.K, info.N,
           (unsigned long long)info.nnz, (unsigned long long)info.stream_bytes);
    sptmm_weights_free(w);
    return 0;
}
