// cli.cpp -- the rcr / ccc command-line programs: the reference's operator surface over the C ABI.
//
// Same flags, same stdout lines and the same per-iteration timing loop as the reference's main()
// (main.cu:38-49 flags, 813-832 banner, 994-1459 loops: launch, synchronise, next), so a script
// written for the reference binaries runs unchanged.  Built twice: -DSPTMM_CLI_RCR gives X row /
// W column / C row major (script/make_rcr.sh:6), -DSPTMM_CLI_CCC all column major
// (script/make_ccc.sh:6).  Host C++ only; the GPU is reached through include/sptmm.h.
//
// Differences, all additive: any shape that meets the constraints is accepted (the reference
// aborts outside a compile-time whitelist, main.cu:1039,1452,1834,1956); `-native` (default 1)
// runs the SpTMM modes on the native encoding instead of the reference layouts; `-check` verifies
// the result against a dense product on the host; `-seed` makes the activations reproducible;
// `-json` adds a machine-readable line on stderr.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "../../include/sptmm.h"

#if defined(SPTMM_CLI_CCC)
static const bool kXCol = true, kCCol = true;
#else
static const bool kXCol = false, kCCol = false;
#endif

namespace {

struct Flags {
    bool cu_blas = false, i2s = false, check = false, json = false;
    uint64_t row_split3_small = 0, row_split_delta2 = 0, M = 32, K = 3072, N = 768, S = 256, L = 1, native = 1;
    uint64_t seed = 0;          // 0 = std::random_device, as the reference (main.cu:788)
    uint32_t iter = 10;
    std::string weights;        // an encoded-weights file (bin/sptmm_encode) to run instead of generating and encoding
};

[[noreturn]] void die(const char *msg)
{
    fprintf(stderr, "%s\n", msg);      // STRICT_ASSERT prints the message and stops (macro.cuh:66)
    exit(EXIT_FAILURE);
}

void must(int rc, const char *what)
{
    if (rc != SPTMM_OK) {
        fprintf(stderr, "%s: %s\n", what, sptmm_last_error());
        exit(EXIT_FAILURE);
    }
}

// gflags syntax: -flag value, -flag=value, --flag=value; booleans also bare or -noflag
Flags parse(int argc, char **argv)
{
    Flags f;
    struct Opt { const char *name; char kind; void *ptr; };
    const Opt opts[] = {
        {"cu_blas", 'b', &f.cu_blas}, {"i2s", 'b', &f.i2s}, {"check", 'b', &f.check}, {"json", 'b', &f.json},
        {"row_split3_small", 'q', &f.row_split3_small}, {"row_split_delta2", 'q', &f.row_split_delta2},
        {"M", 'q', &f.M}, {"K", 'q', &f.K}, {"N", 'q', &f.N}, {"S", 'q', &f.S}, {"L", 'q', &f.L},
        {"native", 'q', &f.native}, {"seed", 'q', &f.seed}, {"iter", 'u', &f.iter}, {"weights", 's', &f.weights},
    };
    for (int i = 1; i < argc; i++) {
        const char *a = argv[i];
        if (a[0] != '-') continue;
        while (*a == '-') a++;
        std::string key(a), val;
        bool has_val = false;
        const size_t eq = key.find('=');
        if (eq != std::string::npos) { val = key.substr(eq + 1); key = key.substr(0, eq); has_val = true; }
        bool found = false;
        for (const Opt &o : opts) {
            if (key == o.name) {
                if (o.kind == 'b' && !has_val) *(bool *)o.ptr = true;
                else {
                    if (!has_val && i + 1 < argc) val = argv[++i];
                    if (o.kind == 's') *(std::string *)o.ptr = val;
                    else if (o.kind == 'b') *(bool *)o.ptr = !(val == "false" || val == "0");
                    else if (o.kind == 'q') *(uint64_t *)o.ptr = strtoull(val.c_str(), nullptr, 10);
                    else *(uint32_t *)o.ptr = (uint32_t)strtoul(val.c_str(), nullptr, 10);
                }
                found = true;
                break;
            }
            if (o.kind == 'b' && key == std::string("no") + o.name) { *(bool *)o.ptr = false; found = true; break; }
        }
        if (!found) {
            fprintf(stderr, "ERROR: unknown command line flag '%s'\n", key.c_str());
            exit(EXIT_FAILURE);
        }
    }
    return f;
}

// main.cu:787-797: round(N(0,5)) clamped to [-127,127]
void make_X(std::vector<int8_t> &X, uint64_t seed)
{
    std::random_device rd;
    std::mt19937 gen(seed ? (uint32_t)seed : rd());
    std::normal_distribution<double> dist(0.0, 5.0);
    for (auto &x : X) x = (int8_t)std::clamp((int)std::round(dist(gen)), -127, 127);
}

struct Device {
    void *X = nullptr, *C = nullptr;
};

double time_loop(uint32_t iter, const std::function<int()> &launch)
{
    const auto t0 = std::chrono::steady_clock::now();
    for (uint32_t i = 0; i < iter; i++) {
        must(launch(), "launch");
        must(sptmm_stream_wait(nullptr), "wait for the default stream");      // the reference synchronises every iteration (main.cu:1456)
    }
    const auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double, std::milli>(t1 - t0).count();
}

void report(const Flags &f, const char *mode, double ms_total, uint64_t stream_bytes, int mismatches)
{
    std::cout << (float)(ms_total / (double)f.iter) << std::endl;      // main.cu:1459
    if (f.json) {
        const double us = ms_total * 1e3 / f.iter;
        const double bytes = (double)stream_bytes + (double)f.M * f.K + (double)f.M * f.N * 4;
        fprintf(stderr, "{\"mode\": \"%s\", \"M\": %llu, \"K\": %llu, \"N\": %llu, \"S\": %llu, \"iter\": %u, "
                "\"us_per_call_sync_each\": %.3f, \"stream_bytes\": %llu, \"effective_GBps\": %.1f, "
                "\"pct_of_8000GBps\": %.2f, \"mismatches\": %d}\n",
                mode, (unsigned long long)f.M, (unsigned long long)f.K, (unsigned long long)f.N,
                (unsigned long long)f.S, f.iter, us, (unsigned long long)stream_bytes, bytes / us / 1e3,
                bytes / us / 1e3 / 80.0, mismatches);
    }
}

// dense product on the host, in the program's own layouts; returns the number of mismatches
int check_result(const Flags &f, const std::vector<int8_t> &W, const std::vector<int8_t> &X, void *C_dev)
{
    std::vector<int32_t> C(f.M * f.N);
    must(sptmm_memcpy_d2h(C.data(), C_dev, C.size() * 4), "copy C back");
    int bad = 0;
    for (uint64_t m = 0; m < f.M; m++)
        for (uint64_t n = 0; n < f.N; n++) {
            int32_t acc = 0;
            for (uint64_t k = 0; k < f.K; k++) {
                const int x = kXCol ? X[k * f.M + m] : X[m * f.K + k];
                acc += x * W[n * f.K + k];
            }
            const int32_t got = kCCol ? C[n * f.M + m] : C[m * f.N + n];
            bad += got != acc;
        }
    fprintf(stderr, "check: %s (%d of %llu outputs differ)\n", bad ? "FAILED" : "OK", bad, (unsigned long long)(f.M * f.N));
    return bad;
}

}  // namespace

int main(int argc, char **argv)
{
    const Flags f = parse(argc, argv);
    // init_ctx (main.cu:85-101); the reference compiles these out with -DNDEBUG, here they hold
    if (f.K >= 65536) die("K should be fit in the maximum of short, since W_M manages indices with short type");
    if (f.S % 2) die("S mod 2 must be 0 s.t. W_map and W_negative becomes the same size");
    if (f.K < f.S) die("K should be bigger than S");
    if (f.M == 0 || f.K == 0 || f.N == 0) die("M, K and N must be positive");
    // mode guards, checked before the device is touched (messages as the reference prints them)
    if (f.cu_blas && (!kXCol || !kCCol)) die("Wrong layout");                                   // main.cu:843-845
    if (f.row_split3_small && f.row_split3_small != 8 && f.row_split3_small != 16 && f.row_split3_small != 32)
        die("Wrong split size");                                                                // main.cu:1039
    if (f.row_split3_small && (f.S / 2) % f.row_split3_small) die("Wrong SPLIT Size");          // main.cu:564
    if (f.row_split_delta2 && f.row_split_delta2 != 32) die("Wrong split size");                // main.cu:1837-1839
    if (f.i2s && kXCol) die("X must be row-major!\n");                                          // main.cu:1852-1854
    if (f.i2s && kCCol) die("C must be row-major!\n");

    int ndev = 0;
    must(sptmm_device_count(&ndev), "cudaGetDeviceCount");
    if (ndev == 0) die("no CUDA device");

    std::vector<int8_t> X(f.M * f.K);
    make_X(X, f.seed);
    Device d;
    must(sptmm_dev_alloc(&d.X, X.size()), "cudaMalloc X");
    must(sptmm_memcpy_h2d(d.X, X.data(), X.size()), "copy X");
    std::cout << "make_X done" << std::endl;
    must(sptmm_dev_alloc(&d.C, f.M * f.N * 4), "cudaMalloc C");

    printf("Compiled on %s at %s\n", __DATE__, __TIME__);
    std::cout << "Start: M=" << f.M << " K=" << f.K << " N=" << f.N << " ITER=" << f.iter << " S=" << f.S
              << " (" << (100.0 - 100.0 * ((float)f.S / (float)f.K)) << "% Sparsity)"
              << " L=" << f.L << " B=" << 8
              << " X_MAJOR=" << (kXCol ? "COL" : "ROW") << " W_MAJOR=COL C_MAJOR=" << (kCCol ? "COL" : "ROW") << std::endl;

    const uint32_t flags = (kXCol ? SPTMM_X_COLMAJOR : 0) | (kCCol ? SPTMM_C_COLMAJOR : 0);
    std::vector<int8_t> W;          // the reference's weights: S/2 of each sign per column (main.cu:248-265)
    auto weights = [&]() -> const std::vector<int8_t> & {
        if (W.empty()) {
            W.resize(f.K * f.N);
            must(sptmm_gen_ternary_fixed((uint32_t)f.K, (uint32_t)f.N, (uint32_t)f.S, W.data()), "generate W");
        }
        return W;
    };
    int rc_total = 0;

    if (f.cu_blas) {
        if (!kXCol || !kCCol) die("Wrong layout");                       // main.cu:843-845
        void *Wd = nullptr;
        must(sptmm_dev_alloc(&Wd, f.K * f.N), "cudaMalloc W");
        must(sptmm_memcpy_h2d(Wd, weights().data(), f.K * f.N), "copy W");
        const double ms = time_loop(f.iter, [&] {
            return sptmm_dense_cublas_gemm((const int8_t *)d.X, (const int8_t *)Wd, (int32_t *)d.C, (uint32_t)f.M, (uint32_t)f.K, (uint32_t)f.N, nullptr);
        });
        const int bad = f.check ? check_result(f, W, X, d.C) : 0;
        report(f, "cu_blas", ms, f.K * f.N, bad);
        rc_total |= bad != 0;
        sptmm_dev_free(Wd);
    }

    auto run_sptmm = [&](const char *mode, uint32_t format, uint32_t split) {
        sptmm_weights *w = nullptr;
        if (!f.weights.empty()) {
            must(sptmm_weights_load(f.weights.c_str(), &w), "weights");
            sptmm_weights_info wi;
            must(sptmm_weights_info_get(w, &wi), "info");
            if (wi.K != f.K || wi.N != f.N) die("the -weights file does not hold a K x N matrix of the -K and -N given");
            if (f.check) weights();       // -check compares with the reference generator's matrix for -K -N -S
        } else {
            must(sptmm_encode(weights().data(), (uint32_t)f.K, (uint32_t)f.N, format, split, (uint32_t)f.S, &w), mode);
        }
        must(sptmm_weights_upload(w), "upload");
        sptmm_weights_info info;
        must(sptmm_weights_info_get(w, &info), "info");
        const double ms = time_loop(f.iter, [&] { return sptmm_gemv(w, d.X, SPTMM_I8, (uint32_t)f.M, d.C, flags, 0, nullptr); });
        const int bad = f.check ? check_result(f, W, X, d.C) : 0;
        report(f, mode, ms, info.stream_bytes, bad);
        rc_total |= bad != 0;
        sptmm_weights_free(w);
    };

    if (f.row_split3_small > 0) {
        const uint64_t sp = f.row_split3_small;
        if (sp != 8 && sp != 16 && sp != 32) die("Wrong split size");     // main.cu:1039
        if ((f.S / 2) % sp) die("Wrong SPLIT Size");                      // main.cu:564
        run_sptmm("row_split3_small", f.native ? SPTMM_FMT_U16_V256 : SPTMM_FMT_U16_DIV, (uint32_t)sp);
    }
    if (f.row_split_delta2 > 0) {
        if (f.row_split_delta2 != 32) die("Wrong split size");            // main.cu:1837-1839
        run_sptmm("row_split_delta2", f.native ? SPTMM_FMT_DELTA_LANE : SPTMM_FMT_DELTA_DIV256, 32);
    }
    if (f.i2s) {
        if (kXCol) die("X must be row-major!\n");                         // main.cu:1852-1854
        if (kCCol) die("C must be row-major!\n");
        if (f.K % 16) die("i2s packs 16 rows per word: K must be a multiple of 16");
        run_sptmm("i2s", SPTMM_FMT_I2S, 0);
    }
    sptmm_dev_free(d.X);
    sptmm_dev_free(d.C);
    return rc_total;
}
