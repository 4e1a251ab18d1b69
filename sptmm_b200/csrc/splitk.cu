// splitk.cu -- a matmul split along K over the GPUs of one node, as an object of the C ABI.
//
// The reference is single-GPU (one device, one stream, main.cu:1861) and splits K only by striding
// lanes over one list (main.cu:581-584); this is the multi-GPU form for matrices whose K is long
// (K up to 28672 in the large sweep).  Rank r holds rows k0..k1 of W and the same slice of every row
// of X; sptmm_gemv_reduce's epilogue adds each column's partial sum to the rank owning the column,
// over NVLink for a peer, so the reduce-scatter needs no kernel of its own.  What this file adds is
// the host side around that call: the shard arithmetic, the per-rank arena (result block + barrier
// flags), and the three stream-ordered phases of a pass
//
//     clear my result block | barrier | accumulate (sptmm_gemv_reduce) | barrier
//
// The barrier is a one-warp kernel: lane r stores this rank's pass counter into rank r's flag array
// (one plain 8-byte store per peer) and then polls its own array until every rank's counter has
// arrived.  Each rank runs on its own GPU, so the kernels of a barrier are co-resident by
// construction; the poll is bounded and raises a status word when it runs out.  Peer memory only
// ever sees plain stores and reductions from this library's kernels.
#include <cuda_runtime.h>

#include <algorithm>

#include "device_common.cuh"
#include "internal.h"

using namespace sptmm;

namespace {

constexpr uint32_t kMaxRanks = 8;
constexpr uint64_t kDefaultPolls = 1ull << 22;

struct BarrierParams {
    unsigned long long *flags[kMaxRanks];   // rank r's flag array (kMaxRanks words), as mapped here
    unsigned long long *own;                // this rank's flag array
    uint32_t *status;
    unsigned long long epoch, limit;
    uint32_t rank, world;
};

__global__ void __launch_bounds__(32, 1) k_rank_barrier(const BarrierParams p)
{
    const uint32_t lane = threadIdx.x;
    // everything earlier on this stream (the cleared block, the additions sent to the peers) is ordered
    // before the flag; a rank that sees the flag sees those
    __threadfence_system();
    if (lane < p.world)
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.flags[lane] + p.rank), "l"(p.epoch) : "memory");
    if (lane < p.world) {
        unsigned long long v = 0, it = 0;
        for (;; it++) {
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p.own + lane) : "memory");
            if (v >= p.epoch) break;
            if (it >= p.limit) { atomicOr(p.status, 1u); break; }      // a rank never arrived: report, do not hang
        }
    }
    __threadfence_system();
}

}  // namespace

struct sptmm_splitk {
    const sptmm_weights *w = nullptr;
    uint32_t dtype = 0, M = 0, rank = 0, world = 1, N = 0, width = 0;
    void *peers[kMaxRanks] = {};             // every rank's result block
    unsigned long long *flags[kMaxRanks] = {};
    void *own_arena = nullptr;               // allocated here when the caller passed none
    uint32_t *d_status = nullptr;
    unsigned long long epoch = 0, limit = kDefaultPolls;
    int device = -1;
};

static size_t block_bytes(uint32_t M, uint32_t N, uint32_t world)
{
    uint32_t mw = 0;
    for (uint32_t r = 0; r < world; r++) mw = std::max(mw, (uint32_t)((uint64_t)N * (r + 1) / world - (uint64_t)N * r / world));
    return ((size_t)M * mw * 4 + 255) & ~(size_t)255;
}

extern "C" int sptmm_splitk_k_range(uint32_t K, uint32_t rank, uint32_t world, uint32_t *k0, uint32_t *k1)
{
    if (!k0 || !k1 || world == 0 || rank >= world) return fail(SPTMM_ERR_INVALID, "splitk_k_range: rank %u of %u", rank, world);
    // contiguous, boundaries on multiples of 16 rows (16-byte loads of int8 activations stay aligned)
    const uint64_t units = ((uint64_t)K + 15) / 16;
    *k0 = (uint32_t)std::min<uint64_t>(K, units * rank / world * 16);
    *k1 = (uint32_t)std::min<uint64_t>(K, units * (rank + 1) / world * 16);
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_col_range(uint32_t N, uint32_t rank, uint32_t world, uint32_t *c0, uint32_t *c1)
{
    if (!c0 || !c1 || world == 0 || rank >= world) return fail(SPTMM_ERR_INVALID, "splitk_col_range: rank %u of %u", rank, world);
    *c0 = (uint32_t)((uint64_t)N * rank / world);           // the rule of sptmm_gemv_reduce's epilogue
    *c1 = (uint32_t)((uint64_t)N * (rank + 1) / world);
    return SPTMM_OK;
}

extern "C" uint64_t sptmm_splitk_arena_bytes(uint32_t M, uint32_t N, uint32_t world)
{
    if (M == 0 || N == 0 || world == 0 || world > kMaxRanks) return 0;
    return block_bytes(M, N, world) + 256;                  // result block | kMaxRanks flag words
}

extern "C" int sptmm_splitk_create(const sptmm_weights *w, uint32_t dtype, uint32_t M, uint32_t rank, uint32_t world,
                                   void *const *arena_peers, sptmm_splitk **out)
{
    if (!w || !out) return fail(SPTMM_ERR_INVALID, "splitk_create: null pointer");
    *out = nullptr;
    if (world == 0 || world > kMaxRanks || rank >= world) return fail(SPTMM_ERR_INVALID, "splitk_create: rank %u of %u (1..8 GPUs of one node)", rank, world);
    if (M == 0 || dtype > SPTMM_F32) return fail(SPTMM_ERR_INVALID, "splitk_create: bad M or dtype");
    if (w->format != SPTMM_FMT_U16_V256 || w->k_tile) return fail(SPTMM_ERR_UNSUPPORTED, "splitk_create: weights must be one native u16 matrix (this rank's K range, or its tile of a K-tiled encoding)");
    if (w->device < 0 || w->dev.empty()) return fail(SPTMM_ERR_STATE, "splitk_create: weights are not uploaded");
    if (w->N < world) return fail(SPTMM_ERR_INVALID, "splitk_create: N=%u columns for %u ranks", w->N, world);
    if (world > 1 && !arena_peers) return fail(SPTMM_ERR_INVALID, "splitk_create: %u ranks need every rank's arena", world);
    int dev = -1;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != w->device) return fail(SPTMM_ERR_STATE, "splitk_create: weights live on device %d, current device is %d", w->device, dev);
    auto s = new sptmm_splitk;
    s->w = w; s->dtype = dtype; s->M = M; s->rank = rank; s->world = world; s->N = w->N; s->device = dev;
    uint32_t c0, c1;
    sptmm_splitk_col_range(w->N, rank, world, &c0, &c1);
    s->width = c1 - c0;
    const size_t blk = block_bytes(M, w->N, world);
    void *own = nullptr;
    if (!arena_peers) {
        const size_t bytes = (size_t)sptmm_splitk_arena_bytes(M, w->N, world);
        cudaError_t e = cudaMalloc(&s->own_arena, bytes);
        if (e == cudaSuccess) e = cudaMemset(s->own_arena, 0, bytes);
        if (e != cudaSuccess) { cudaFree(s->own_arena); delete s; return fail(SPTMM_ERR_CUDA, "splitk_create: arena: %s", cudaGetErrorString(e)); }
        own = s->own_arena;
    }
    for (uint32_t r = 0; r < world; r++) {
        unsigned char *a = static_cast<unsigned char *>(arena_peers ? arena_peers[r] : own);
        if (!a || (reinterpret_cast<uintptr_t>(a) & 255)) { sptmm_splitk_free(s); return fail(SPTMM_ERR_INVALID, "splitk_create: arena of rank %u is null or not 256-byte aligned", r); }
        s->peers[r] = a;
        s->flags[r] = reinterpret_cast<unsigned long long *>(a + blk);
    }
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&s->d_status), 4);
    if (e == cudaSuccess) e = cudaMemset(s->d_status, 0, 4);
    if (e != cudaSuccess) { sptmm_splitk_free(s); return fail(SPTMM_ERR_CUDA, "splitk_create: status word: %s", cudaGetErrorString(e)); }
    *out = s;
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_free(sptmm_splitk *s)
{
    if (!s) return SPTMM_OK;
    if (s->d_status) cudaFree(s->d_status);
    if (s->own_arena) cudaFree(s->own_arena);
    delete s;
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_clear(sptmm_splitk *s, void *stream)
{
    if (!s) return fail(SPTMM_ERR_INVALID, "splitk_clear: null handle");
    SPTMM_CUDA_TRY(cudaMemsetAsync(s->peers[s->rank], 0, (size_t)s->M * s->width * 4, static_cast<cudaStream_t>(stream)));
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_barrier(sptmm_splitk *s, void *stream)
{
    if (!s) return fail(SPTMM_ERR_INVALID, "splitk_barrier: null handle");
    if (s->world == 1) return SPTMM_OK;
    BarrierParams p{};
    for (uint32_t r = 0; r < s->world; r++) p.flags[r] = s->flags[r];
    p.own = s->flags[s->rank];
    p.status = s->d_status;
    p.epoch = ++s->epoch;
    p.limit = s->limit;
    p.rank = s->rank; p.world = s->world;
    k_rank_barrier<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    SPTMM_CUDA_TRY(cudaGetLastError());
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_accumulate(sptmm_splitk *s, const void *X_slice, uint32_t flags, void *stream)
{
    if (!s || !X_slice) return fail(SPTMM_ERR_INVALID, "splitk_accumulate: null pointer");
    return sptmm_gemv_reduce(s->w, X_slice, s->dtype, s->M, s->peers, s->world, flags, 0, stream);
}

extern "C" int sptmm_splitk_forward(sptmm_splitk *s, const void *X_slice, uint32_t flags, void *stream)
{
    int rc = sptmm_splitk_clear(s, stream);
    if (rc == SPTMM_OK) rc = sptmm_splitk_barrier(s, stream);          // nobody adds into a block that is not cleared yet
    if (rc == SPTMM_OK) rc = sptmm_splitk_accumulate(s, X_slice, flags, stream);
    if (rc == SPTMM_OK) rc = sptmm_splitk_barrier(s, stream);          // every rank's additions have landed
    return rc;
}

extern "C" int sptmm_splitk_output(const sptmm_splitk *s, void **C, uint32_t *width)
{
    if (!s || !C) return fail(SPTMM_ERR_INVALID, "splitk_output: null pointer");
    *C = s->peers[s->rank];
    if (width) *width = s->width;
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_status(sptmm_splitk *s, uint32_t *status)
{
    if (!s || !status) return fail(SPTMM_ERR_INVALID, "splitk_status: null pointer");
    uint32_t word = 0, gemv = 0;
    SPTMM_CUDA_TRY(cudaMemcpy(&word, s->d_status, 4, cudaMemcpyDeviceToHost));       // waits for the device
    const int rc = sptmm_gemv_status(s->w, &gemv);
    if (rc != SPTMM_OK) return rc;
    *status = word | (gemv ? 2u : 0u);
    return SPTMM_OK;
}

extern "C" int sptmm_splitk_set_wait_limit(sptmm_splitk *s, uint64_t polls)
{
    if (!s) return fail(SPTMM_ERR_INVALID, "splitk_set_wait_limit: null handle");
    s->limit = polls ? polls : kDefaultPolls;
    return SPTMM_OK;
}
