// ref_harness.cu -- runs the SpTMM reference's OWN kernels, unmodified, and dumps what they produce.
//
// TEST INFRASTRUCTURE ONLY.  The reference binary prints a time and never reads its result
// back, so it cannot serve as an oracle as shipped.  This translation unit includes the
// reference's main.cu where it lies (its main() renamed), then drives prepareW_map and the
// SpTMM kernels on seeded activations and writes inputs, encodings and results to files,
// which become the golden fixtures the CPU restatement and the CUDA library are pinned to.
//
//   ref_harness readme <reference flags...>   run the reference's main() as shipped
//   ref_harness dump <outdir> [case ...]      run the built-in cases (all if none named)
//   ref_harness list                          print case names
//
// Built by oracle/Makefile into oracle/_ref/ (never committed).
#define main sptmm_reference_main
#include "main.cu"
#undef main
#undef M
#undef K
#undef N
#undef S
#undef L

#include <string>
#include <vector>
#include <cstdio>
#include <sys/stat.h>

namespace {

struct Case {
    const char *name;
    const char *mode;                 // "split3" or "delta"
    uint32_t m, k, n, s, split;
    bool full_dump;                   // small case: every array is written in full
    void (*launch)(const char *X, const void *wp, const void *wn, int *C);
};

template <uint M_, uint K_, uint N_, uint S_, uint SPLIT>
void launch_split3(const char *X, const void *wp, const void *wn, int *C)
{
    rowWiseSplit3Small4<M_, K_, N_, S_, SPLIT><<<dim3(N_ / (32 / SPLIT), M_, 1), dim3(SPLIT, 32 / SPLIT, 1)>>>(
        X, (const unsigned short *)wp, (const unsigned short *)wn, C);
}
template <uint M_, uint K_, uint N_, uint S_>
void launch_delta2(const char *X, const void *wp, const void *wn, int *C)
{
    rowWiseSplit2DeltaSmallAsync2<M_, K_, N_, S_, 32><<<dim3(N_, M_, 1), 32>>>(
        X, (const unsigned char *)wp, (const unsigned char *)wn, C);
}
template <uint M_, uint K_, uint N_, uint S_>
void launch_delta3(const char *X, const void *wp, const void *wn, int *C)
{
    rowWiseSplit2DeltaSmallAsync3<M_, K_, N_, S_, 32><<<dim3(N_, M_, 1), 32>>>(
        X, (const unsigned char *)wp, (const unsigned char *)wn, C);
}

const Case kCases[] = {
    {"s3_m1_k256_n32_s128_sp8",   "split3", 1, 256, 32, 128, 8,  true,  launch_split3<1, 256, 32, 128, 8>},
    {"s3_m1_k256_n32_s128_sp16",  "split3", 1, 256, 32, 128, 16, true,  launch_split3<1, 256, 32, 128, 16>},
    {"s3_m1_k256_n32_s128_sp32",  "split3", 1, 256, 32, 128, 32, true,  launch_split3<1, 256, 32, 128, 32>},
    {"s3_m4_k256_n32_s128_sp32",  "split3", 4, 256, 32, 128, 32, true,  launch_split3<4, 256, 32, 128, 32>},
    {"s3_m8_k512_n48_s256_sp8",   "split3", 8, 512, 48, 256, 8,  true,  launch_split3<8, 512, 48, 256, 8>},
    {"dl_m1_k1024_n32_s512",      "delta",  1, 1024, 32, 512, 32, true, launch_delta2<1, 1024, 32, 512>},
    {"dl_m1_k1024_n32_s384",      "delta",  1, 1024, 32, 384, 32, true, launch_delta3<1, 1024, 32, 384>},
    {"dl_m4_k1024_n32_s512",      "delta",  4, 1024, 32, 512, 32, true, launch_delta2<4, 1024, 32, 512>},
    {"s3_m1_k6912_n2560_s4096_sp32", "split3", 1, 6912, 2560, 4096, 32, false, launch_split3<1, 6912, 2560, 4096, 32>},
    {"s3_m1_k6912_n2560_s4096_sp16", "split3", 1, 6912, 2560, 4096, 16, false, launch_split3<1, 6912, 2560, 4096, 16>},
    {"s3_m1_k6912_n2560_s4096_sp8",  "split3", 1, 6912, 2560, 4096, 8,  false, launch_split3<1, 6912, 2560, 4096, 8>},
    {"s3_m4_k6912_n2560_s4096_sp32", "split3", 4, 6912, 2560, 4096, 32, false, launch_split3<4, 6912, 2560, 4096, 32>},
    {"s3_m1_k6912_n2560_s4608_sp32", "split3", 1, 6912, 2560, 4608, 32, false, launch_split3<1, 6912, 2560, 4608, 32>},
    {"dl_m1_k6912_n2560_s4096",   "delta",  1, 6912, 2560, 4096, 32, false, launch_delta2<1, 6912, 2560, 4096>},
    {"dl_m1_k6912_n2560_s4608",   "delta",  1, 6912, 2560, 4608, 32, false, launch_delta2<1, 6912, 2560, 4608>},
    {"dl_m1_k6912_n2560_s3456",   "delta",  1, 6912, 2560, 3456, 32, false, launch_delta3<1, 6912, 2560, 3456>},
    {"dl_m1_k6912_n2560_s1728",   "delta",  1, 6912, 2560, 1728, 32, false, launch_delta3<1, 6912, 2560, 1728>},
    {"dl_m4_k6912_n2560_s4096",   "delta",  4, 6912, 2560, 4096, 32, false, launch_delta2<4, 6912, 2560, 4096>},
};

uint64_t fnv1a64(const void *p, size_t n)
{
    const unsigned char *b = (const unsigned char *)p;
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 0x100000001b3ull; }
    return h;
}

// int8 activations, uniform on [-127,127], xorshift32 stream (seed 0 -> golden-ratio constant).
void seeded_x(std::vector<char> &x, uint32_t seed)
{
    uint32_t s = seed ? seed : 0x9E3779B9u;
    for (auto &v : x) v = (char)((int)(xorshift32(&s) % 255u) - 127);
}

struct DevBuf {
    void *p = nullptr; size_t bytes = 0;
    void alloc(size_t b) { bytes = b ? b : 1; checkCudaErrors(cudaMalloc(&p, bytes)); checkCudaErrors(cudaMemset(p, 0, bytes)); }
    ~DevBuf() { if (p) cudaFree(p); }
};

FILE *g_manifest = nullptr;
bool g_first = true;

void emit(const std::string &dir, const Case &c, const char *array, const char *dtype,
          const DevBuf &d, size_t bytes, bool write_file)
{
    std::vector<unsigned char> h(bytes);
    checkCudaErrors(cudaMemcpy(h.data(), d.p, bytes, cudaMemcpyDeviceToHost));
    uint64_t hash = fnv1a64(h.data(), bytes);
    if (write_file) {
        std::string path = dir + "/" + c.name + "." + array + ".bin";
        FILE *f = fopen(path.c_str(), "wb");
        if (!f) { perror(path.c_str()); exit(1); }
        fwrite(h.data(), 1, bytes, f);
        fclose(f);
    }
    fprintf(g_manifest, "%s\n  {\"case\": \"%s\", \"array\": \"%s\", \"dtype\": \"%s\", \"bytes\": %zu, "
            "\"fnv1a64\": \"%016llx\", \"file\": %s}",
            g_first ? "" : ",", c.name, array, dtype, bytes, (unsigned long long)hash,
            write_file ? "true" : "false");
    g_first = false;
}

float time_loop(int iters, bool sync_each, const std::function<void(int)> &fn)
{
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
    for (int i = 0; i < 5; i++) fn(i);
    cudaDeviceSynchronize();
    cudaEventRecord(a);
    for (int i = 0; i < iters; i++) { fn(i); if (sync_each) cudaDeviceSynchronize(); }
    cudaEventRecord(b);
    cudaEventSynchronize(b);
    float ms = 0; cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a); cudaEventDestroy(b);
    return ms * 1000.0f / (float)iters;   // microseconds per call
}

void run_case(const std::string &dir, const Case &c, FILE *timing)
{
    FLAGS_M = c.m; FLAGS_K = c.k; FLAGS_N = c.n; FLAGS_S = c.s; FLAGS_L = 1;
    init_ctx();
    const size_t m = c.m, k = c.k, n = c.n, s = c.s, h = s / 2, b256 = 256 * n * CEIL_DIV(h, 256);

    std::vector<char> x(m * k);
    seeded_x(x, 1u + (uint32_t)(m * 131 + k));
    DevBuf X, C; X.alloc(m * k); C.alloc(4 * m * n);
    checkCudaErrors(cudaMemcpy(X.p, x.data(), m * k, cudaMemcpyHostToDevice));

    // The 31 output arrays of prepareW_map with the sizes main() gives them (main.cu:914-970).
    DevBuf work, map, mapn, sb, sbn, sd, sdn, d2, d2n, acc, accn, vv, vc, vi, vi16,
           d32, d32n, d8, d8n, d16, d16n, d64, d64n, d128, d128n, d256, d256n, d512, d512n,
           dl256, dl256n, dl32, dl32n;
    work.alloc(k * n); map.alloc(2 * h * n); mapn.alloc(2 * h * n);
    sb.alloc(2 * 128 * n); sbn.alloc(2 * 128 * n); sd.alloc(h * n); sdn.alloc(h * n);
    d2.alloc(h * n); d2n.alloc(h * n); acc.alloc(h * n); accn.alloc(h * n);
    vv.alloc(2 * n); vc.alloc(2 * 2 * n); vi.alloc(2 * s * n); vi16.alloc(2 * s * n);
    d32.alloc(2 * h * n); d32n.alloc(2 * h * n); d8.alloc(2 * h * n); d8n.alloc(2 * h * n);
    d16.alloc(2 * h * n); d16n.alloc(2 * h * n); d64.alloc(2 * h * n); d64n.alloc(2 * h * n);
    d128.alloc(2 * h * n); d128n.alloc(2 * h * n); d256.alloc(2 * b256); d256n.alloc(2 * b256);
    d512.alloc(2 * h * n); d512n.alloc(2 * h * n);
    dl256.alloc(b256); dl256n.alloc(b256); dl32.alloc(h * n); dl32n.alloc(h * n);

    prepareW_map<<<c.n / 16, 16>>>(
        (char *)work.p, (unsigned short *)map.p, (unsigned short *)mapn.p,
        (unsigned short *)sb.p, (unsigned short *)sbn.p, (unsigned char *)sd.p, (unsigned char *)sdn.p,
        (unsigned char *)d2.p, (unsigned char *)d2n.p, (unsigned char *)acc.p, (unsigned char *)accn.p,
        (char *)vv.p, (unsigned short *)vc.p, (unsigned short *)vi.p, (unsigned short *)vi16.p,
        (unsigned short *)d32.p, (unsigned short *)d32n.p, (unsigned short *)d8.p, (unsigned short *)d8n.p,
        (unsigned short *)d16.p, (unsigned short *)d16n.p, (unsigned short *)d64.p, (unsigned short *)d64n.p,
        (unsigned short *)d128.p, (unsigned short *)d128n.p, (unsigned short *)d256.p, (unsigned short *)d256n.p,
        (unsigned short *)d512.p, (unsigned short *)d512n.p,
        (unsigned char *)dl256.p, (unsigned char *)dl256n.p, (unsigned char *)dl32.p, (unsigned char *)dl32n.p,
        ctx_v);
    checkCudaErrors(cudaGetLastError());
    checkCudaErrors(cudaDeviceSynchronize());

    const bool delta = std::string(c.mode) == "delta";
    const DevBuf *wp = delta ? &dl256 : (c.split == 32 ? &d32 : c.split == 16 ? &d16 : &d8);
    const DevBuf *wn = delta ? &dl256n : (c.split == 32 ? &d32n : c.split == 16 ? &d16n : &d8n);
    const size_t wbytes = delta ? b256 : 2 * h * n;

    c.launch((const char *)X.p, wp->p, wn->p, (int *)C.p);
    checkCudaErrors(cudaGetLastError());
    checkCudaErrors(cudaDeviceSynchronize());

    const bool f = c.full_dump;
    emit(dir, c, "X", "i8", X, m * k, true);
    emit(dir, c, "C", "i32", C, 4 * m * n, true);
    emit(dir, c, "W_dense", "i8", work, k * n, f);
    emit(dir, c, "W_map", "u16", map, 2 * h * n, f);
    emit(dir, c, "W_map_negative", "u16", mapn, 2 * h * n, f);
    emit(dir, c, "W_map_32_div", "u16", d32, 2 * h * n, f);
    emit(dir, c, "W_map_negative_32_div", "u16", d32n, 2 * h * n, f);
    emit(dir, c, "W_map_16_div", "u16", d16, 2 * h * n, f);
    emit(dir, c, "W_map_negative_16_div", "u16", d16n, 2 * h * n, f);
    emit(dir, c, "W_map_8_div", "u16", d8, 2 * h * n, f);
    emit(dir, c, "W_map_negative_8_div", "u16", d8n, 2 * h * n, f);
    emit(dir, c, "W_map_delta2_div256", "u8", dl256, b256, f);
    emit(dir, c, "W_map_negative_delta2_div256", "u8", dl256n, b256, f);

    if (!c.full_dump && timing) {
        // Reference kernel time on this GPU: warm (one weight copy, L2-resident), cold (rotating
        // distinct copies whose total exceeds L2), and the reference's own sync-per-call style.
        const int copies = (int)std::min<size_t>(24, std::max<size_t>(2, (400u << 20) / (2 * wbytes)));
        std::vector<DevBuf> rp(copies), rn(copies);
        for (int i = 0; i < copies; i++) {
            rp[i].alloc(wbytes); rn[i].alloc(wbytes);
            cudaMemcpy(rp[i].p, wp->p, wbytes, cudaMemcpyDeviceToDevice);
            cudaMemcpy(rn[i].p, wn->p, wbytes, cudaMemcpyDeviceToDevice);
        }
        float warm = time_loop(2000, false, [&](int) { c.launch((const char *)X.p, wp->p, wn->p, (int *)C.p); });
        float cold = time_loop(2000, false, [&](int i) { c.launch((const char *)X.p, rp[i % copies].p, rn[i % copies].p, (int *)C.p); });
        float sync = time_loop(2000, true,  [&](int) { c.launch((const char *)X.p, wp->p, wn->p, (int *)C.p); });
        fprintf(timing, "{\"case\": \"%s\", \"weight_bytes\": %zu, \"copies\": %d, \"us_warm\": %.3f, "
                "\"us_cold\": %.3f, \"us_sync_each\": %.3f}\n", c.name, 2 * wbytes, copies, warm, cold, sync);
        fflush(timing);
    }
}

}  // namespace

int main(int argc, char **argv)
{
    if (argc >= 2 && std::string(argv[1]) == "readme") {
        return sptmm_reference_main(argc - 1, argv + 1);
    }
    if (argc >= 2 && std::string(argv[1]) == "list") {
        for (const Case &c : kCases) printf("%s\n", c.name);
        return 0;
    }
    if (argc >= 3 && std::string(argv[1]) == "dump") {
        std::string dir = argv[2];
        mkdir(dir.c_str(), 0755);
        g_manifest = fopen((dir + "/manifest.json").c_str(), "w");
        FILE *timing = fopen((dir + "/reference_timing.jsonl").c_str(), "w");
        if (!g_manifest || !timing) { perror("open"); return 1; }
        fprintf(g_manifest, "[");
        for (const Case &c : kCases) {
            bool want = argc == 3;
            for (int i = 3; i < argc; i++) if (std::string(argv[i]) == c.name) want = true;
            if (!want) continue;
            run_case(dir, c, timing);
            printf("done %s\n", c.name);
        }
        fprintf(g_manifest, "\n]\n");
        fclose(g_manifest); fclose(timing);
        return 0;
    }
    fprintf(stderr, "usage: %s readme <flags> | dump <outdir> [case...] | list\n", argv[0]);
    return 2;
}
