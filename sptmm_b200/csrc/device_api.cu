// device_api.cu -- the C ABI's device side: upload, launch dispatch, host-buffer convenience
// call, raw-pointer entry points and small helpers.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <string>

#include "device_common.cuh"

namespace sptmm {

const Tune &tune()
{
    // Two 256-thread CTAs per SM, four blocks per warp in registers and a ~50 KB footprint per
    // CTA: measured best on B200 both for one stream (5.7 us per 6912x2560 GEMV) and for
    // independent calls on several streams (3.2 us, the HBM copy rate), because up to four
    // CTAs of neighbouring calls fit one SM and overlap their stream / gather phases.
    static const Tune t = {(int)tuning_knob("SPTMM_TUNE_CTAS_PER_SM", 2), (int)tuning_knob("SPTMM_TUNE_THREADS", 256),
                           (int)tuning_knob("SPTMM_TUNE_PREFETCH", 4), (int)tuning_knob("SPTMM_TUNE_SMEM_KB", 43)};
    return t;
}

#ifdef SPTMM_TUNING
long tuning_knob(const char *name, long dflt)
{
    const char *e = getenv(name);
    return e ? atol(e) : dflt;
}
#endif

static void free_host_slot(sptmm_weights::HostSlot &h)
{
    if (h.dev_x) cudaFree(h.dev_x);
    if (h.pin_x) cudaFreeHost(h.pin_x);
    if (h.pin_c) cudaFreeHost(h.pin_c);
    if (h.pin_status) cudaFreeHost(h.pin_status);
    if (h.stream) cudaStreamDestroy((cudaStream_t)h.stream);
    h = sptmm_weights::HostSlot();
}

static void free_device_side(sptmm_weights *w)
{
    if (w->device >= 0) {
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(w->device);
        for (auto &rep : w->dev) for (void *p : rep) if (p) cudaFree(p);
        if (w->plan.d_status) cudaFree(w->plan.d_status);
        for (auto &h : w->slots) {
            if (h.busy && h.stream) cudaStreamSynchronize((cudaStream_t)h.stream);
            free_host_slot(h);
        }
        cudaSetDevice(cur);
    }
    w->dev.clear();
    w->plan = LaunchPlan();
    w->plan_wide = LaunchPlan();
    w->device = -1;
}

// Give each of `grid` CTAs a contiguous run of whole columns holding about total/grid blocks.
// off = the 2N+1 list boundaries of a native-format matrix.
// With col_align = 2 every boundary falls on an even column (steps that sum column pairs).
void plan_columns(const uint32_t *off, uint32_t N, uint32_t grid, std::vector<uint32_t> &cta_blk,
                  std::vector<uint32_t> &cta_col, uint32_t &max_cols, uint32_t &max_cta_blocks,
                  uint32_t col_align)
{
    const uint64_t total = off[2 * (size_t)N];
    cta_blk.clear(); cta_col.clear();
    max_cols = 1; max_cta_blocks = 0;
    uint32_t c = 0;
    for (uint32_t i = 0; i < grid; i++) {
        const uint64_t target = total * (i + 1) / grid;
        uint32_t c1 = c;
        if (i + 1 == grid) c1 = N;
        else {
            while (c1 < N && off[2 * (size_t)(c1 + 1)] <= target) c1++;
            // take one more column if that lands closer to the target
            if (c1 < N && (int64_t)off[2 * (size_t)(c1 + 1)] - (int64_t)target < (int64_t)target - (int64_t)off[2 * (size_t)c1]) c1++;
            if (col_align > 1) c1 = std::min(N, std::max(c, (c1 + col_align - 1) / col_align * col_align));
        }
        cta_blk.push_back(off[2 * (size_t)c]);
        cta_col.push_back(c);
        max_cols = std::max(max_cols, c1 - c);
        max_cta_blocks = std::max(max_cta_blocks, off[2 * (size_t)c1] - off[2 * (size_t)c]);
        c = c1;
    }
    cta_blk.push_back(off[2 * (size_t)N]);
    cta_col.push_back(N);
}

static void make_plan(sptmm_weights *w)
{
    LaunchPlan &pl = w->plan;
    const Tune &t = tune();
    pl.grid = std::min<uint32_t>(w->sm_count * t.ctas_per_sm, kMaxPlanCtas);
    pl.threads = t.threads;
    plan_columns((const uint32_t *)w->arrays[1].data.data(), w->N, pl.grid, pl.cta_blk, pl.cta_col, pl.max_cols, pl.max_cta_blocks);
    LaunchPlan &pw = w->plan_wide;
    pw.grid = std::min<uint32_t>(w->sm_count, kMaxPlanCtas);
    pw.threads = 512;
    plan_columns((const uint32_t *)w->arrays[1].data.data(), w->N, pw.grid, pw.cta_blk, pw.cta_col, pw.max_cols, pw.max_cta_blocks);
}

}  // namespace sptmm

using namespace sptmm;

extern "C" int sptmm_weights_upload_replicas(sptmm_weights *w, uint32_t copies)
{
    if (!w) return fail(SPTMM_ERR_INVALID, "weights_upload: null handle");
    if (copies == 0 || copies > 4096) return fail(SPTMM_ERR_INVALID, "weights_upload: copies=%u", copies);
    if (w->k_tile) {                        // a K-tiled matrix: every tile, to the same device
        for (sptmm_weights *t : w->tiles) {
            const int rc = sptmm_weights_upload_replicas(t, copies);
            if (rc != SPTMM_OK) return rc;
        }
        w->device = w->tiles.empty() ? -1 : w->tiles[0]->device;
        return SPTMM_OK;
    }
    free_device_side(w);
    int dev = 0, sms = 0;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    SPTMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    w->device = dev;
    w->sm_count = (uint32_t)sms;
    w->dev.assign(copies, std::vector<void *>(w->arrays.size(), nullptr));
    for (uint32_t r = 0; r < copies; r++)
        for (size_t a = 0; a < w->arrays.size(); a++) {
            const size_t bytes = std::max<size_t>(w->arrays[a].data.size(), 16);
            cudaError_t e = cudaMalloc(&w->dev[r][a], bytes);
            if (e == cudaSuccess)
                e = cudaMemcpy(w->dev[r][a], w->arrays[a].data.data(), w->arrays[a].data.size(), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                free_device_side(w);
                return fail(SPTMM_ERR_CUDA, "weights_upload: %s", cudaGetErrorString(e));
            }
        }
    if (w->format == SPTMM_FMT_U16_V256 || w->format == SPTMM_FMT_DELTA_LANE) {
        make_plan(w);
        cudaError_t e = cudaMalloc(&w->plan.d_status, 16);
        if (e == cudaSuccess) e = cudaMemset(w->plan.d_status, 0, 16);
        if (e != cudaSuccess) {
            free_device_side(w);
            return fail(SPTMM_ERR_CUDA, "weights_upload: %s", cudaGetErrorString(e));
        }
    }
    return SPTMM_OK;
}

extern "C" int sptmm_weights_upload(sptmm_weights *w) { return sptmm_weights_upload_replicas(w, 1); }

extern "C" int sptmm_weights_free(sptmm_weights *w)
{
    if (!w) return SPTMM_OK;
    for (sptmm_weights *t : w->tiles) sptmm_weights_free(t);
    w->tiles.clear();
    free_device_side(w);
    delete w;
    return SPTMM_OK;
}

static int gemv_dispatch(const sptmm_weights *w, const void *X, uint32_t dtype, uint32_t M, void *C,
                         uint32_t flags, uint32_t replica, void *stream, uint32_t *status)
{
    if (!w || !X || !C) return fail(SPTMM_ERR_INVALID, "gemv: null pointer");
    if (M == 0) return fail(SPTMM_ERR_INVALID, "gemv: M must be at least 1");
    if (dtype > SPTMM_F32) return fail(SPTMM_ERR_INVALID, "gemv: unknown dtype %u", dtype);
    if (w->k_tile) {
        // tile after tile on the stream: the first stores, the others add; each reads its own K range of X
        const size_t es = dtype_size(dtype);
        for (size_t t = 0; t < w->tiles.size(); t++) {
            const sptmm_weights *tw = w->tiles[t];
            if (tw->device < 0 || tw->dev.empty()) return fail(SPTMM_ERR_STATE, "gemv: tile %zu of the K-tiled weights is not uploaded", t);
            if (replica >= tw->dev.size()) return fail(SPTMM_ERR_INVALID, "gemv: replica %u of %zu", replica, tw->dev.size());
            const size_t k0 = t * (size_t)w->k_tile;
            const char *xt = static_cast<const char *>(X) + ((flags & SPTMM_X_COLMAJOR) ? k0 * M : k0) * es;
            GemvArgs a{tw, tw->dev[replica].data(), xt, C, dtype, M, flags, stream};
            a.status = status; a.ldx = w->K; a.accumulate = t > 0;
            const int rc = launch_native_u16(a);
            if (rc != SPTMM_OK) return rc;
        }
        return SPTMM_OK;
    }
    if (w->device < 0 || w->dev.empty()) return fail(SPTMM_ERR_STATE, "gemv: weights are not uploaded");
    if (replica >= w->dev.size()) return fail(SPTMM_ERR_INVALID, "gemv: replica %u of %zu", replica, w->dev.size());
    int dev = -1;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != w->device) return fail(SPTMM_ERR_STATE, "gemv: weights live on device %d, current device is %d", w->device, dev);
    const void *const *arr = w->dev[replica].data();
    GemvArgs a{w, arr, X, C, dtype, M, flags, stream};
    a.status = status;
    switch (w->format) {
        case SPTMM_FMT_U16_V256: return launch_native_u16(a);
        case SPTMM_FMT_DELTA_LANE: return launch_native_delta(a);
        case SPTMM_FMT_I2S: return launch_i2s(a);
        case SPTMM_FMT_U16_DIV:
            return launch_div(X, (const uint16_t *)arr[0], (const uint16_t *)arr[1], C, dtype, M, w->K, w->N, w->S,
                              w->split, flags, stream);
        case SPTMM_FMT_DELTA_DIV256:
            return launch_delta256(X, (const uint8_t *)arr[0], (const uint8_t *)arr[1], C, dtype, M, w->K, w->N, w->S,
                                   flags, stream);
    }
    return fail(SPTMM_ERR_UNSUPPORTED, "gemv: format %u", w->format);
}

extern "C" int sptmm_gemv(const sptmm_weights *w, const void *X, uint32_t dtype, uint32_t M, void *C,
                          uint32_t flags, uint32_t replica, void *stream)
{
    return gemv_dispatch(w, X, dtype, M, C, flags, replica, stream, nullptr);
}

extern "C" int sptmm_gemv_scaled(const sptmm_weights *w, const int8_t *X, uint32_t M, float *C, const float *row_scale,
                                 float w_scale, uint32_t flags, uint32_t replica, void *stream)
{
    if (!w || !X || !C) return fail(SPTMM_ERR_INVALID, "gemv_scaled: null pointer");
    if (M == 0) return fail(SPTMM_ERR_INVALID, "gemv_scaled: M must be at least 1");
    if ((w->format != SPTMM_FMT_U16_V256 && w->format != SPTMM_FMT_DELTA_LANE) || w->k_tile)
        return fail(SPTMM_ERR_UNSUPPORTED, "gemv_scaled: weights must be one matrix in a native format");
    if (w->device < 0 || w->dev.empty()) return fail(SPTMM_ERR_STATE, "gemv_scaled: weights are not uploaded");
    if (replica >= w->dev.size()) return fail(SPTMM_ERR_INVALID, "gemv_scaled: replica %u of %zu", replica, w->dev.size());
    int dev = -1;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != w->device) return fail(SPTMM_ERR_STATE, "gemv_scaled: weights live on device %d, current device is %d", w->device, dev);
    GemvArgs a{w, w->dev[replica].data(), X, C, SPTMM_I8, M, flags, stream};
    a.scaled = true; a.row_scale = row_scale; a.out_scale = w_scale;
    return w->format == SPTMM_FMT_U16_V256 ? launch_native_u16(a) : launch_native_delta(a);
}

extern "C" int sptmm_gemv_reduce(const sptmm_weights *w, const void *X, uint32_t dtype, uint32_t M,
                                 void *const *C_peers, uint32_t n_peers, uint32_t flags, uint32_t replica,
                                 void *stream)
{
    if (!w || !X || !C_peers) return fail(SPTMM_ERR_INVALID, "gemv_reduce: null pointer");
    if (n_peers == 0 || n_peers > 8) return fail(SPTMM_ERR_INVALID, "gemv_reduce: n_peers=%u (1..8 GPUs of one node)", n_peers);
    for (uint32_t r = 0; r < n_peers; r++)
        if (!C_peers[r]) return fail(SPTMM_ERR_INVALID, "gemv_reduce: no output buffer for rank %u", r);
    if (M == 0 || dtype > SPTMM_F32) return fail(SPTMM_ERR_INVALID, "gemv_reduce: bad M or dtype");
    if (w->format != SPTMM_FMT_U16_V256 || w->k_tile) return fail(SPTMM_ERR_UNSUPPORTED, "gemv_reduce: weights must be one native u16 matrix (for a K-tiled one, the rank's own tile)");
    if (flags & SPTMM_C_COLMAJOR) return fail(SPTMM_ERR_UNSUPPORTED, "gemv_reduce: the per-rank outputs are row-major");
    if (w->N < n_peers) return fail(SPTMM_ERR_INVALID, "gemv_reduce: N=%u columns for %u ranks", w->N, n_peers);
    if (w->device < 0 || w->dev.empty()) return fail(SPTMM_ERR_STATE, "gemv_reduce: weights are not uploaded");
    if (replica >= w->dev.size()) return fail(SPTMM_ERR_INVALID, "gemv_reduce: replica %u of %zu", replica, w->dev.size());
    int dev = -1;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != w->device) return fail(SPTMM_ERR_STATE, "gemv_reduce: weights live on device %d, current device is %d", w->device, dev);
    GemvArgs a{w, w->dev[replica].data(), X, C_peers[0], dtype, M, flags, stream};
    a.C_peers = C_peers;
    a.n_peers = n_peers;
    return launch_native_u16(a);
}

// The per-call kernels' bounded waits raise a word in device memory when they run out (the kernel
// then finishes with whatever it has); this reads it back.
static int read_gemv_status(const sptmm_weights *w, uint32_t *word)
{
    *word = 0;
    if (!w->plan.d_status) return SPTMM_OK;            // formats whose kernels have no waits
    SPTMM_CUDA_TRY(cudaMemcpy(word, w->plan.d_status, 4, cudaMemcpyDeviceToHost));
    return SPTMM_OK;
}

extern "C" int sptmm_gemv_status(const sptmm_weights *w, uint32_t *status)
{
    if (!w || !status) return fail(SPTMM_ERR_INVALID, "gemv_status: null pointer");
    if (w->k_tile) {                        // a K-tiled matrix: any tile's word
        *status = 0;
        for (const sptmm_weights *t : w->tiles) {
            uint32_t word = 0;
            const int rc = sptmm_gemv_status(t, &word);
            if (rc != SPTMM_OK) return rc;
            *status |= word;
        }
        return SPTMM_OK;
    }
    if (w->device < 0) return fail(SPTMM_ERR_STATE, "gemv_status: weights are not uploaded");
    int dev = -1;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != w->device) return fail(SPTMM_ERR_STATE, "gemv_status: weights live on device %d, current device is %d", w->device, dev);
    SPTMM_CUDA_TRY(cudaDeviceSynchronize());
    return read_gemv_status(w, status);
}

extern "C" int sptmm_gemv_host_wait(sptmm_weights *w, uint32_t slot)
{
    if (!w || slot >= sptmm_weights::kHostSlots) return fail(SPTMM_ERR_INVALID, "gemv_host_wait: bad handle or slot %u", slot);
    sptmm_weights::HostSlot &h = w->slots[slot];
    if (!h.busy) return SPTMM_OK;
    cudaStream_t st = (cudaStream_t)h.stream;
    // a short busy wait first: for a call of a few microseconds polling the stream returns sooner
    // than the blocking wait does (replaying copy + kernel as one instantiated graph was tried as
    // well: no gain at M=1, slower at M=4; so was a completion word in pinned host memory, stored
    // by the kernel's last CTA behind system-wide fences and polled here without driver calls:
    // 31 us against 28 us per blocking call, 6.8 us against 4.7 us with sixteen calls in flight)
    cudaError_t qe = cudaErrorNotReady;
    for (int spin = 0; spin < 20000 && qe == cudaErrorNotReady; spin++) qe = cudaStreamQuery(st);
    if (qe == cudaErrorNotReady) qe = cudaStreamSynchronize(st);
    h.busy = false;
    if (qe != cudaSuccess) return fail(SPTMM_ERR_CUDA, "gemv_host: %s", cudaGetErrorString(qe));
    // The status word sits in mapped pinned memory for host-buffer calls (see _async), so this check
    // is a host load: a call whose bounded wait ran out must not hand back partial sums as a result.
    if (h.pin_status && *(volatile uint32_t *)h.pin_status != 0)
        return fail(SPTMM_ERR_STATE, "gemv_host: a bounded wait in the kernel ran out (status %u); the result was dropped",
                    *(volatile uint32_t *)h.pin_status);
    memcpy(h.user_c, h.pin_c, h.user_c_bytes);
    return SPTMM_OK;
}

extern "C" int sptmm_gemv_host_async(sptmm_weights *w, const void *X_host, uint32_t dtype, uint32_t M, void *C_host,
                                     uint32_t flags, uint32_t replica, uint32_t slot)
{
    if (!w || !X_host || !C_host) return fail(SPTMM_ERR_INVALID, "gemv_host: null pointer");
    if (M == 0 || dtype > SPTMM_F32) return fail(SPTMM_ERR_INVALID, "gemv_host: bad M or dtype");
    if (slot >= sptmm_weights::kHostSlots) return fail(SPTMM_ERR_INVALID, "gemv_host: slot %u of %u", slot, sptmm_weights::kHostSlots);
    if (w->device < 0) return fail(SPTMM_ERR_STATE, "gemv_host: weights are not uploaded");
    sptmm_weights::HostSlot &h = w->slots[slot];
    if (h.busy) {                              // the slot's previous call has to deliver its result first
        const int rc = sptmm_gemv_host_wait(w, slot);
        if (rc != SPTMM_OK) return rc;
    }
    const size_t xb = (size_t)M * w->K * dtype_size(dtype), cb = (size_t)M * w->N * 4;
    if (!h.stream) {
        cudaStream_t s;
        SPTMM_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        h.stream = s;
    }
    if (xb > h.x_bytes) {
        if (h.dev_x) cudaFree(h.dev_x);
        if (h.pin_x) cudaFreeHost(h.pin_x);
        h.dev_x = h.pin_x = nullptr; h.x_bytes = 0;
        SPTMM_CUDA_TRY(cudaMalloc(&h.dev_x, xb));
        SPTMM_CUDA_TRY(cudaMallocHost(&h.pin_x, xb));
        h.x_bytes = xb;
    }
    if (cb > h.c_bytes) {
        // The result goes straight into mapped pinned host memory: every output element is
        // written exactly once, so the kernel's own stores replace a device buffer plus a copy
        // engine operation (dev_c is the device's address of pin_c, not an allocation).
        if (h.pin_c) cudaFreeHost(h.pin_c);
        h.dev_c = h.pin_c = nullptr; h.c_bytes = 0;
        SPTMM_CUDA_TRY(cudaHostAlloc(&h.pin_c, cb, cudaHostAllocMapped));
        SPTMM_CUDA_TRY(cudaHostGetDevicePointer(&h.dev_c, h.pin_c, 0));
        h.c_bytes = cb;
    }
    if (!h.pin_status) {
        SPTMM_CUDA_TRY(cudaHostAlloc(&h.pin_status, 16, cudaHostAllocMapped));
        SPTMM_CUDA_TRY(cudaHostGetDevicePointer(&h.dev_status, h.pin_status, 0));
    }
    *(volatile uint32_t *)h.pin_status = 0;
    cudaStream_t st = (cudaStream_t)h.stream;
    memcpy(h.pin_x, X_host, xb);
    // X does go through a device copy: every CTA reads all of it, and reads of host memory are
    // not cached on the device (measured: 87 us per call with X left in pinned host memory).
    // Letting the kernel's first CTA fetch the pinned X for the others (no copy-engine operation)
    // was measured too: 25.8 us against 24.0 us per blocking call -- a PCIe read inside the
    // kernel is slower than the copy engine's.
    SPTMM_CUDA_TRY(cudaMemcpyAsync(h.dev_x, h.pin_x, xb, cudaMemcpyHostToDevice, st));
    const int rc = gemv_dispatch(w, h.dev_x, dtype, M, h.dev_c, flags & ~(uint32_t)SPTMM_LAUNCH_PDL, replica, st,
                                 (uint32_t *)h.dev_status);
    if (rc != SPTMM_OK) return rc;
    h.user_c = C_host; h.user_c_bytes = cb; h.busy = true;
    return SPTMM_OK;
}

extern "C" int sptmm_gemv_host(sptmm_weights *w, const void *X_host, uint32_t dtype, uint32_t M, void *C_host,
                               uint32_t flags, uint32_t replica)
{
    const int rc = sptmm_gemv_host_async(w, X_host, dtype, M, C_host, flags, replica, 0);
    return rc != SPTMM_OK ? rc : sptmm_gemv_host_wait(w, 0);
}

extern "C" int sptmm_gemv_host_batch(sptmm_weights *w, uint32_t n, const void *const *X_hosts, void *const *C_hosts,
                                     const uint32_t *replicas, uint32_t dtype, uint32_t M, uint32_t flags,
                                     uint32_t slot0, uint32_t nslots)
{
    if (!w || (n && (!X_hosts || !C_hosts))) return fail(SPTMM_ERR_INVALID, "gemv_host_batch: null pointer");
    if (nslots == 0 || slot0 >= sptmm_weights::kHostSlots || nslots > sptmm_weights::kHostSlots - slot0)
        return fail(SPTMM_ERR_INVALID, "gemv_host_batch: slots %u..%u of %u", slot0, slot0 + nslots, sptmm_weights::kHostSlots);
    int rc = SPTMM_OK;
    for (uint32_t i = 0; i < n && rc == SPTMM_OK; i++)
        rc = sptmm_gemv_host_async(w, X_hosts[i], dtype, M, C_hosts[i], flags, replicas ? replicas[i] : 0, slot0 + i % nslots);
    std::string first_error = rc != SPTMM_OK ? sptmm_last_error() : "";
    for (uint32_t s = 0; s < nslots; s++) {
        const int wrc = sptmm_gemv_host_wait(w, slot0 + s);
        if (rc == SPTMM_OK && wrc != SPTMM_OK) { rc = wrc; first_error = sptmm_last_error(); }
    }
    return rc == SPTMM_OK ? SPTMM_OK : fail(rc, "%s", first_error.c_str());
}

extern "C" int sptmm_row_split3_small(const int8_t *X, const uint16_t *W_pos_div, const uint16_t *W_neg_div,
                                      int32_t *C, uint32_t M, uint32_t K, uint32_t N, uint32_t S,
                                      uint32_t split, void *stream)
{
    return launch_div(X, W_pos_div, W_neg_div, C, SPTMM_I8, M, K, N, S, split, 0, stream);
}

extern "C" int sptmm_row_split_delta2(const int8_t *X, const uint8_t *W_pos_delta, const uint8_t *W_neg_delta,
                                      int32_t *C, uint32_t M, uint32_t K, uint32_t N, uint32_t S,
                                      uint32_t split, void *stream)
{
    if (split != 32) return fail(SPTMM_ERR_INVALID, "Wrong split size");     // main.cu:1837-1839
    return launch_delta256(X, W_pos_delta, W_neg_delta, C, SPTMM_I8, M, K, N, S, 0, stream);
}

#ifdef SPTMM_TUNING
extern "C" int sptmm_set_trace_buffer(void *dev_ptr)
{
    set_trace_buffer((unsigned long long *)dev_ptr);
    return SPTMM_OK;
}
#endif

extern "C" int sptmm_device_count(int *count)
{
    if (!count) return fail(SPTMM_ERR_INVALID, "device_count: null pointer");
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) { *count = 0; return fail(SPTMM_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e)); }
    return SPTMM_OK;
}
extern "C" int sptmm_set_device(int device) { SPTMM_CUDA_TRY(cudaSetDevice(device)); return SPTMM_OK; }
extern "C" int sptmm_dev_alloc(void **ptr, uint64_t bytes)
{
    if (!ptr) return fail(SPTMM_ERR_INVALID, "dev_alloc: null pointer");
    SPTMM_CUDA_TRY(cudaMalloc(ptr, bytes ? bytes : 1));
    return SPTMM_OK;
}
extern "C" int sptmm_dev_free(void *ptr) { SPTMM_CUDA_TRY(cudaFree(ptr)); return SPTMM_OK; }
extern "C" int sptmm_memcpy_h2d(void *dst, const void *src, uint64_t bytes)
{
    SPTMM_CUDA_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    return SPTMM_OK;
}
extern "C" int sptmm_memcpy_d2h(void *dst, const void *src, uint64_t bytes)
{
    SPTMM_CUDA_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return SPTMM_OK;
}
extern "C" int sptmm_device_sync(void) { SPTMM_CUDA_TRY(cudaDeviceSynchronize()); return SPTMM_OK; }

extern "C" int sptmm_stream_wait(void *stream)
{
    // for work of a few microseconds, asking whether the stream is done returns sooner than the
    // blocking wait does; after a while fall back to it
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaErrorNotReady;
    for (int spin = 0; spin < 20000 && e == cudaErrorNotReady; spin++) e = cudaStreamQuery(st);
    if (e == cudaErrorNotReady) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(SPTMM_ERR_CUDA, "stream_wait: %s", cudaGetErrorString(e));
    return SPTMM_OK;
}
