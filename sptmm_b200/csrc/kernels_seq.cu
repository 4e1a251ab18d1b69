// kernels_seq.cu -- one persistent kernel that runs a whole sequence of ternary matmuls.
//
// No counterpart in the reference, which launches one kernel per matmul and synchronises the
// host after each (main.cu:994-1458).  A kernel boundary costs more than the 3 us a 21 MB
// matrix needs to stream from HBM, so here a single cooperative launch (one CTA per SM) walks
// a list of steps; each step is C = X*W for one encoded matrix (native u16 format).
//
//  - Weights: every warp owns, for every step, the same contiguous slice of blocks the
//    per-call kernel gives it, and runs a private ring of 4 KB slots in shared memory filled by
//    bulk copies (cp.async.bulk + mbarrier).  The ring is refilled as slots are consumed and
//    runs ahead across step boundaries, so the next matrix streams from HBM while this one is
//    still being gathered and while the CTAs synchronise.
//  - Dependencies: a step may wait for an earlier step to have finished on all CTAs (its input
//    is that step's output).  Each CTA adds 1 to the step's counter after its results are
//    visible; waiters poll the counter with acquire loads.  Every wait is bounded: if one runs
//    out, the kernel raises a status word, stops waiting and runs to the end.
//  - Activations: int8 rows are staged transposed in shared memory as in the per-call kernel.
//    A step can instead take int32 outputs of earlier steps (optionally the sum of two) and
//    quantise them on the fly to int8 with a per-row absmax scale, which fuses the activation
//    quantiser between the layers of a stack into the matmul.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "device_common.cuh"

namespace sptmm {

#ifndef SPTMM_SEQ_SLOT_BLOCKS
#define SPTMM_SEQ_SLOT_BLOCKS 8
#endif
constexpr uint32_t kMaxSlotBlocks = SPTMM_SEQ_SLOT_BLOCKS;   // 512-byte blocks per ring slot (4 KB streams best;
                                                             // smaller only when the X tile leaves less room)
constexpr uint32_t kMaxPeers = 8;                            // GPUs of one node

struct SeqDesc {
    const uint4 *idx;            // encoded blocks of this step's matrix
    const uint32_t *blk_off;     // its 2N+1 list boundaries
    const void *X;               // activations: int8 (x_kind 0) or int32 (x_kind 1), row stride ldx
    const void *X2;              // optional second int32 source added to X (x_kind 1)
    int32_t *C;                  // output, row stride ldc
    float *scale_out;            // optional: absmax/127 per row of the quantised input
    uint32_t K, N, ldx, ldx2, ldc, uniform_nbl, x_kind;
    int32_t dep;                 // step that must be complete before this one reads X, or -1
    int32_t *Cp[kMaxPeers];      // multi-GPU: this shard's place in every rank's output buffer
    // Tagged exchange (x_kind 2 consumers).  A tagged output word is (tag << 24) | (value & 0xffffff)
    // with tag = seq_tag(run, m, j): j counts the steps of one run that write this buffer, m is
    // their number, so two successive writes of a word never carry the same tag and a reader can
    // tell a fresh value from the one it replaces without any flag or fence.
    uint32_t out_tag_m, out_tag_j;   // this step's output: m == 0 -> plain int32
    uint32_t in_tag_m, in_tag_j;     // x_kind 2: the tag of the step that produces X (and X2)
    uint32_t release;                // 1: bump the step counter after the output is stored
    uint32_t c_kind;                 // 1: the output is the sum of each pair of neighbouring columns (N/2 values)
    uint32_t want_amax;              // 1: a later x_kind 3 step wants this step's row maxima recorded
    // Producer-side quantiser (an x_kind 4 reader): this step turns its output columns
    // [q_0, q_0 + q_n) -- counted from its first own column, so q_0 may be negative on a rank whose
    // shard starts further right -- into int8 itself, in two hand-overs: every CTA publishes the row
    // maxima of its own columns (amax1, then amax2 between GPUs), and once a CTA knows the rows'
    // maxima over all columns it rounds ITS columns and stores them, three rows to a tagged word, in
    // every rank's copy of the packed buffer.  The offsets count bytes from the start of a rank's
    // synchronisation area (the same on every rank).
    uint32_t q_n;                    // 0: off
    int32_t q_0;
    uint32_t q_off, amax1_off, amax2_off;
    float *q_scale_out;              // optional: absmax/127 per row (the reader's scale_out)
};

constexpr uint32_t kAmaxStride = 256;            // row maxima: [16 rows][kAmaxStride CTAs] per step
__host__ __device__ inline uint32_t packed_words(uint32_t M) { return (M + 2) / 3; }   // tagged words per column: three rows each

constexpr uint32_t kPollLimit = 1u << 20;        // reloads of one stale word before giving up

__device__ __forceinline__ uint32_t seq_tag(uint32_t run_mod, uint32_t m, uint32_t j) { return 1u + (run_mod * m + j) % 255u; }
__device__ __forceinline__ int untag(int v) { return (v << 8) >> 8; }          // sign-extend the low 24 bits

// (poll_batch below is the form the staging code uses: it keeps a thread's reloads in flight together)
// a load other CTAs' (and, with sys, other GPUs') plain stores become visible to
__device__ __forceinline__ int ld_fresh(const int32_t *p, bool sys)
{
    int v;
    if (sys) asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    else asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int4 ld_fresh4(const int4 *p, bool sys)
{
    int4 v;
    if (sys) asm volatile("ld.relaxed.sys.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else asm volatile("ld.relaxed.gpu.global.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// v[j] was loaded from base[tid + j*nt] (entries at or beyond K are not used).  Round by round,
// reload the words that do not carry `tag` yet -- all reloads of a round in flight at once -- until
// none is stale (bounded); then strip the tags.
template <int V>
__device__ __forceinline__ void poll_batch(int (&v)[V], const int32_t *base, uint32_t K, uint32_t tid, uint32_t nt,
                                           uint32_t tag, bool sys, bool &ok)
{
    for (uint32_t it = 0; ok; it++) {
        bool stale = false;
#pragma unroll
        for (int j = 0; j < V; j++) {
            const uint32_t k = tid + j * nt;
            if (k < K && ((uint32_t)v[j] >> 24) != tag) { stale = true; v[j] = ld_fresh(base + k, sys); }
        }
        if (!stale) break;
        if (it >= kPollLimit) ok = false;
    }
#pragma unroll
    for (int j = 0; j < V; j++) v[j] = untag(v[j]);
}


struct SeqParams {
    const SeqDesc *desc;
    const uint32_t *cta_blk;     // [nsteps][G+1]
    const uint32_t *cta_col;     // [nsteps][G+1]
    unsigned long long *counters;           // this rank's step counters
    unsigned long long *counter_peers[kMaxPeers];   // every rank's (peer-mapped); used when n_peers > 0
    uint32_t n_peers;            // 0: single GPU
    uint32_t *status;
#ifdef SPTMM_TUNING
    unsigned long long *trace;   // optional timestamps for kernel timelines (tuning build only)
#endif
    unsigned long long target;   // counters[s] >= target  <=>  step s finished in this run
    uint32_t nsteps, M, max_cols, ring_slots, xs_bytes, G;
    uint32_t slot_blocks;        // 512-byte blocks per ring slot
    uint32_t one;                // always 1: a multiplier the compiler cannot fold (LaneAcc::add)
    uint32_t run_mod;            // run number mod 255 (tags of the tagged exchange change every run)
    // Row maxima for x_kind 3: amax[(parity * nsteps + step) * 16 + row], on this rank and (peer-mapped)
    // on every rank; a run uses the half `run_parity` and clears the other half for the next run.
    uint32_t *amax;
    uint32_t *amax_peers[kMaxPeers];
    uint32_t run_parity;
    uint32_t my_rank;
    // x_kind 5 (settled exchange): two local counters per step, and two buffers (by step parity) for
    // the finished int8 tile every CTA then fetches with one bulk copy
    unsigned long long *settle;
    unsigned char *xq;
    uint32_t xq_stride;
    unsigned long long target_local;   // settle[i] >= target_local  <=>  every CTA of THIS GPU has arrived in this run
    uint32_t poll_limit;               // reloads of a counter (or of a settled-exchange word) before a wait gives up
};

#ifdef SPTMM_TUNING
// Timestamp for the optional trace.  A bare read of %globaltimer is hoisted by the assembler
// (it was seen moving above barriers); guarding it with a predicate computed from a volatile
// shared-memory load pins it behind whatever that load is ordered after.
__device__ __forceinline__ unsigned long long seq_ns(const volatile uint32_t *anchor)
{
    const uint32_t v = *anchor;
    unsigned long long t;
    asm volatile("{ .reg .pred p; setp.ne.u32 p, %1, 0xdeadbeef; @p mov.u64 %0, %globaltimer; @!p mov.u64 %0, 0; }"
                 : "=l"(t) : "r"(v) : "memory");
    return t;
}
#endif

// Every CTA's timestamp at a point inside the input stage, for steps 100..103 (tuning build only).
#ifdef SPTMM_TUNING
#define SEQ_MARK_BY(prm, step, slot, anchor, who)                                                            \
    do {                                                                                                     \
        if ((prm).trace != nullptr && threadIdx.x == (who) && (step) >= 100 && (step) < 104)                  \
            (prm).trace[5120 + (slot) * 1024 + ((step) - 100) * 256 + blockIdx.x] = seq_ns(anchor);           \
    } while (0)
#define SEQ_MARK(prm, step, slot, anchor)                                                                   \
    do {                                                                                                     \
        if ((prm).trace != nullptr && threadIdx.x == 33 && (step) >= 100 && (step) < 104)                     \
            (prm).trace[5120 + (slot) * 1024 + ((step) - 100) * 256 + blockIdx.x] = seq_ns(anchor);           \
    } while (0)
#else
#define SEQ_MARK(prm, step, slot, anchor) do { } while (0)
#define SEQ_MARK_BY(prm, step, slot, anchor, who) do { } while (0)
#endif

// 16 bytes of a ring slot by shared-space address
__device__ __forceinline__ uint4 lds_vec(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

__device__ __forceinline__ void seq_bulk_fetch(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Non-blocking variant for the producer warp, whose lanes poll different barriers: a blocking
// try_wait in one lane would stall the copies of all the others.
__device__ __forceinline__ bool seq_bounded_poll(uint32_t bar, uint32_t parity)
{
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < (1u << 26) && !done; spin++)
        asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

__device__ __forceinline__ bool seq_bounded_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < (1u << 22) && !done; spin++)
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

// Tiles of several rows hold x+128 as unsigned bytes (the form LaneAcc's packed sums expect).
template <int MT> constexpr uint32_t kTileBias = MT > 1 ? 0x80808080u : 0u;
template <int MT> __device__ __forceinline__ int8_t tile_byte(int q) { return (int8_t)(MT > 1 ? (q ^ 0x80) : q); }

// absmax/127 of the rows the current step's input stage quantised (1 for int8 inputs): every input
// stage leaves it here for the de-quantising epilogue (c_kind 2)
__shared__ float seq_xscale_s[16];

constexpr int kRedInts = 32 + 16 * 16 + 16;      // scratch ints behind the column sums (see stage_x_quant_rows)

__device__ __forceinline__ int absmax4(int4 v) { return max(max(abs(v.x), abs(v.y)), max(abs(v.z), abs(v.w))); }
__device__ __forceinline__ int quant1(int v, float scale)
{
    return max(-127, min(127, __float2int_rn((float)v * scale)));
}

// All CTAs stage the same activations at the same time.  Walking them in the same order makes every
// SM ask the same L2 slice at the same moment (measured: 2 TB/s in all, a third of what L2 gives);
// each CTA therefore starts at its own offset and wraps around.
__device__ __forceinline__ uint32_t cta_rotation(uint32_t n) { return (uint32_t)(((uint64_t)blockIdx.x * n) / gridDim.x); }
__device__ __forceinline__ uint32_t rotated(uint32_t i, uint32_t rot, uint32_t n) { return i + rot < n ? i + rot : i + rot - n; }

// The quantiser for tiles of 4 or 16 rows, all rows at once.  Pass 1: every thread walks the
// rows in 16-byte pieces (all rows' loads of a piece in flight together) and keeps one running
// absmax per row; warps combine them through shared memory (two barriers in all).  Pass 2 reads
// the values again (they are L2-resident), rounds them and writes whole tile words: the four
// rows of a group are packed into one word per k.  Needs K, the row strides and the pointers
// to be multiples of four ints; red must hold kRedInts ints.
template <int MT>
__device__ __forceinline__ void stage_x_quant_rows(unsigned char *xs, const SeqDesc &d, uint32_t M, int *red, bool write_scale,
                                                   uint32_t tag, bool sys, bool &ok)
{
    // tag != 0: the sources hold tagged words; the first pass waits for each to become current
    auto stale4 = [&](const int4 &v) {
        return ((uint32_t)v.x >> 24) != tag || ((uint32_t)v.y >> 24) != tag || ((uint32_t)v.z >> 24) != tag || ((uint32_t)v.w >> 24) != tag;
    };
    // A thread's loads go out a group of GR rows at a time: each group is one round trip to L2, and
    // the round trips -- not bandwidth -- are what the quantiser costs, so 16-row tiles use groups
    // of eight rows (32 registers in flight).
    constexpr int GR = MT == 16 ? 8 : 4;
    // rows row0..row0+GR-1 of one source at piece q; with a tag, reload the stale ones round by
    // round (the reloads of a round in flight together) until all are current
    auto fetch_rows = [&](const int4 *S, uint32_t ld, int row0, uint32_t q, int4 (&v)[GR]) {
#pragma unroll
        for (int r = 0; r < GR; r++)
            v[r] = (uint32_t)(row0 + r) < M ? __ldcg(S + (size_t)(row0 + r) * ld + q) : make_int4(0, 0, 0, 0);
        if (tag) {
            for (uint32_t it = 0; ok; it++) {
                bool stale = false;
#pragma unroll
                for (int r = 0; r < GR; r++)
                    if ((uint32_t)(row0 + r) < M && stale4(v[r])) { stale = true; v[r] = ld_fresh4(S + (size_t)(row0 + r) * ld + q, sys); }
                if (!stale) break;
                if (it >= kPollLimit) ok = false;
            }
#pragma unroll
            for (int r = 0; r < GR; r++) v[r] = make_int4(untag(v[r].x), untag(v[r].y), untag(v[r].z), untag(v[r].w));
        }
    };
    auto again4 = [&](const int4 *p) {
        int4 v = __ldcg(p);
        if (tag) v = make_int4(untag(v.x), untag(v.y), untag(v.z), untag(v.w));
        return v;
    };
    static_assert(MT % 4 == 0, "row tiles of 4 or 16");
    const int4 *A = reinterpret_cast<const int4 *>(d.X);
    const int4 *B = reinterpret_cast<const int4 *>(d.X2);
    const uint32_t tid = threadIdx.x, nt = 512, lane = tid & 31, warp = tid >> 5;      // consumer threads only
    const uint32_t quads = d.K / 4, lda = d.ldx / 4, ldb = d.ldx2 / 4;
    int *part = red + 32;                     // [16 warps][16 rows]
    int *amax_s = red + 32 + 256;             // [16 rows]

    int am[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) am[m] = 0;
    const uint32_t rot = cta_rotation(quads);

    for (uint32_t q0 = tid; q0 < quads; q0 += nt) {
        const uint32_t q = rotated(q0, rot, quads);
#pragma unroll
        for (int g = 0; g < MT / GR; g++) {
            int4 v[GR];
            fetch_rows(A, lda, GR * g, q, v);
            if (B) {
                int4 b[GR];
                fetch_rows(B, ldb, GR * g, q, b);
#pragma unroll
                for (int r = 0; r < GR; r++) { v[r].x += b[r].x; v[r].y += b[r].y; v[r].z += b[r].z; v[r].w += b[r].w; }
            }
#pragma unroll
            for (int r = 0; r < GR; r++) am[GR * g + r] = max(am[GR * g + r], absmax4(v[r]));
        }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const int r = __reduce_max_sync(0xffffffffu, am[m]);
        if (lane == 0) part[warp * 16 + m] = r;
    }
    asm volatile("bar.sync 1, 512;" ::: "memory");
    if (warp < (uint32_t)MT) {                // warp m folds row m
        const int r = __reduce_max_sync(0xffffffffu, lane < 16 ? part[lane * 16 + warp] : 0);
        if (lane == 0) amax_s[warp] = r;
    }
    asm volatile("bar.sync 1, 512;" ::: "memory");
    float scale[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const int a = amax_s[m];
        scale[m] = a ? 127.0f / (float)a : 0.0f;
        if (tid == (uint32_t)m) seq_xscale_s[m] = (float)a / 127.0f;
        if (write_scale && d.scale_out && tid == (uint32_t)m && (uint32_t)m < M) d.scale_out[m] = (float)a / 127.0f;
    }

    for (uint32_t q0 = tid; q0 < quads; q0 += nt) {
        const uint32_t q = rotated(q0, rot, quads);
#pragma unroll
        for (int g8 = 0; g8 < MT / GR; g8++) {
            int4 w[GR];
#pragma unroll
            for (int r = 0; r < GR; r++) {
                const int m = GR * g8 + r;
                w[r] = (uint32_t)m < M ? again4(A + (size_t)m * lda + q) : make_int4(0, 0, 0, 0);
            }
            if (B) {
#pragma unroll
                for (int r = 0; r < GR; r++) {
                    const int m = GR * g8 + r;
                    if ((uint32_t)m < M) {
                        const int4 b = again4(B + (size_t)m * ldb + q);
                        w[r].x += b.x; w[r].y += b.y; w[r].z += b.z; w[r].w += b.w;
                    }
                }
            }
#pragma unroll
          for (int h = 0; h < GR / 4; h++) {
            const int g = g8 * (GR / 4) + h;
            const int4 (&v)[4] = *reinterpret_cast<const int4 (*)[4]>(&w[4 * h]);
            uint32_t o[4];                    // o[i]: rows 4g..4g+3 at k = 4q+i
#define SPTMM_PACK4(f) ((uint32_t)(quant1(v[0].f, scale[4 * g]) & 0xff) | ((uint32_t)(quant1(v[1].f, scale[4 * g + 1]) & 0xff) << 8) | \
                        ((uint32_t)(quant1(v[2].f, scale[4 * g + 2]) & 0xff) << 16) | ((uint32_t)(quant1(v[3].f, scale[4 * g + 3]) & 0xff) << 24))
            o[0] = SPTMM_PACK4(x) ^ 0x80808080u;
            o[1] = SPTMM_PACK4(y) ^ 0x80808080u;
            o[2] = SPTMM_PACK4(z) ^ 0x80808080u;
            o[3] = SPTMM_PACK4(w) ^ 0x80808080u;
#undef SPTMM_PACK4
            if constexpr (MT == 4) {
                *reinterpret_cast<uint4 *>(xs + (size_t)q * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++)
                    *reinterpret_cast<uint32_t *>(xs + ((size_t)q * 4 + i) * MT + 4 * g) = o[i];
            }
          }
        }
    }
    if (tid < (uint32_t)MT) xs[(size_t)d.K * MT + tid] = 0x80;        // the zero row
}

// One complete int32 row -> int8 tile, 16 bytes per load, the values kept in registers between
// the absmax and the rounding; `tagged`: the words carry a tag byte to strip.  The trip count is
// uniform over the CTA, so rows far shorter than the register budget cost no idle instructions.
// Needs K % 4 == 0, A 16-byte aligned, K <= 14336.
__device__ __forceinline__ bool row_fits_vec(const void *A, uint32_t K)
{
    return (K & 3) == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 && K <= 7u * 4u * 512u;
}
__device__ __forceinline__ void quant_row_vec(unsigned char *xs, const int32_t *A, uint32_t K, int *red, bool tagged, float *scale_out)
{
    constexpr int V4 = 7;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nt = 512;
    const uint32_t quads = K / 4, nv = (quads + nt - 1) / nt;
    int4 v[V4];
    int amax = 0;
#pragma unroll
    for (int j = 0; j < V4; j++) {
        if ((uint32_t)j < nv) {
            const uint32_t q = tid + j * nt;
            v[j] = q < quads ? __ldcg(reinterpret_cast<const int4 *>(A) + q) : make_int4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int j = 0; j < V4; j++) {
        if ((uint32_t)j < nv) {
            if (tagged) v[j] = make_int4((v[j].x << 8) >> 8, (v[j].y << 8) >> 8, (v[j].z << 8) >> 8, (v[j].w << 8) >> 8);
            amax = max(amax, max(max(abs(v[j].x), abs(v[j].y)), max(abs(v[j].z), abs(v[j].w))));
        }
    }
    amax = __reduce_max_sync(0xffffffffu, amax);
    if (lane == 0) red[warp] = amax;
    asm volatile("bar.sync 1, 512;" ::: "memory");
    amax = lane < 16 ? red[lane] : 0;
    amax = __reduce_max_sync(0xffffffffu, amax);
    const float scale = amax ? 127.0f / (float)amax : 0.0f;
    auto q1 = [&](int x) { return (uint32_t)max(-127, min(127, __float2int_rn((float)x * scale))) & 0xffu; };
#pragma unroll
    for (int j = 0; j < V4; j++) {
        if ((uint32_t)j < nv) {
            const uint32_t q = tid + j * nt;
            if (q < quads) reinterpret_cast<uint32_t *>(xs)[q] = q1(v[j].x) | (q1(v[j].y) << 8) | (q1(v[j].z) << 16) | (q1(v[j].w) << 24);
        }
    }
    if (tid == 0) xs[K] = 0;
    if (tid == 0) seq_xscale_s[0] = (float)amax / 127.0f;
    if (scale_out && tid == 0) scale_out[0] = (float)amax / 127.0f;
}

// int32 rows (optionally the sum of two sources) -> int8 with a per-row absmax scale:
// q = clamp(rint(v * (127 / amax)), -127, 127), all in fp32; amax == 0 gives zeros.
template <int MT, bool TAGGED>
__device__ __forceinline__ void stage_x_quant(unsigned char *xs, const SeqDesc &d, uint32_t M, int *red, bool write_scale,
                                              uint32_t tag_in, bool sys, bool &ok)
{
    const uint32_t tag = TAGGED ? tag_in : 0u;       // a kernel without tagged steps carries none of the waiting code
    // tag != 0: the sources hold tagged words (see SeqDesc); wait for each to become current
    auto first = [&](const int32_t *p) {          // rows too long for the one-pass form: one word at a time
        int v = __ldcg(p);
        if (tag) {
            for (uint32_t it = 0; ok && ((uint32_t)v >> 24) != tag; it++) {
                if (it >= kPollLimit) { ok = false; break; }
                v = ld_fresh(p, sys);
            }
            v = untag(v);
        }
        return v;
    };
    auto again = [&](const int32_t *p) { const int v = __ldcg(p); return tag ? untag(v) : v; };
    if constexpr (MT >= 4) {
        if ((d.K & 3) == 0 && (d.ldx & 3) == 0 && (d.ldx2 & 3) == 0 && (reinterpret_cast<uintptr_t>(d.X) & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(d.X2) & 15) == 0) {
            stage_x_quant_rows<MT>(xs, d, M, red, write_scale, tag, sys, ok);
            return;
        }
    }
    const int32_t *A = reinterpret_cast<const int32_t *>(d.X);
    const int32_t *B = reinterpret_cast<const int32_t *>(d.X2);
    if constexpr (MT == 1) {
        if (!tag && !B && M >= 1 && row_fits_vec(A, d.K)) {          // the common case: one finished row
            quant_row_vec(xs, A, d.K, red, false, (write_scale && d.scale_out) ? d.scale_out : nullptr);
            return;
        }
    }
    int8_t *dst = reinterpret_cast<int8_t *>(xs);
    const uint32_t tid = threadIdx.x, nt = 512, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;   // consumer threads only
    constexpr int V = 28;                      // values a thread keeps per row: covers K <= 14336
    if (d.K <= (uint32_t)V * nt) {
        // One pass: the row's values stay in registers between the absmax and the rounding, so
        // the input is read once and a row costs one load latency and one barrier.
        for (uint32_t m = 0; m < (uint32_t)MT; m++) {
            if (m >= M) {
                for (uint32_t k = tid; k < d.K; k += nt) dst[(size_t)k * MT + m] = tile_byte<MT>(0);
                continue;
            }
            int v[V];
#pragma unroll
            for (int j = 0; j < V; j++) {
                const uint32_t k = tid + j * nt;
                v[j] = k < d.K ? __ldcg(A + (size_t)m * d.ldx + k) : 0;          // all loads in flight, then the tag checks
            }
            if (tag) poll_batch<V>(v, A + (size_t)m * d.ldx, d.K, tid, nt, tag, sys, ok);
            if (B && !tag) {
#pragma unroll
                for (int j = 0; j < V; j++) {
                    const uint32_t k = tid + j * nt;
                    if (k < d.K) v[j] += __ldcg(B + (size_t)m * d.ldx2 + k);
                }
            } else if (B) {
                constexpr int VB = 14;                            // second source in batches: loads first, checks after
#pragma unroll
                for (int j0 = 0; j0 < V; j0 += VB) {
                    int b[VB];
#pragma unroll
                    for (int j = 0; j < VB; j++) {
                        const uint32_t k = tid + (j0 + j) * nt;
                        b[j] = k < d.K ? __ldcg(B + (size_t)m * d.ldx2 + k) : 0;
                    }
                    const uint32_t done = (uint32_t)j0 * nt;
                    poll_batch<VB>(b, B + (size_t)m * d.ldx2 + done, d.K > done ? d.K - done : 0u, tid, nt, tag, sys, ok);
#pragma unroll
                    for (int j = 0; j < VB; j++) v[j0 + j] += b[j];
                }
            }
            int amax = 0;
#pragma unroll
            for (int j = 0; j < V; j++) amax = max(amax, abs(v[j]));
            amax = __reduce_max_sync(0xffffffffu, amax);
            int *slot = red + (m & 1) * 16;                       // alternate halves: one barrier per row
            if (lane == 0) slot[warp] = amax;
            asm volatile("bar.sync 1, 512;" ::: "memory");
            amax = 0;
            for (uint32_t w = 0; w < nwarps; w++) amax = max(amax, slot[w]);
            const float scale = amax ? 127.0f / (float)amax : 0.0f;
#pragma unroll
            for (int j = 0; j < V; j++) {
                const uint32_t k = tid + j * nt;
                if (k < d.K) {
                    int q = __float2int_rn((float)v[j] * scale);
                    q = max(-127, min(127, q));
                    dst[(size_t)k * MT + m] = tile_byte<MT>(q);
                }
            }
            if (tid == 0) seq_xscale_s[m] = (float)amax / 127.0f;
            if (write_scale && d.scale_out && tid == 0) d.scale_out[m] = (float)amax / 127.0f;
        }
        if (tid < (uint32_t)MT) dst[(size_t)d.K * MT + tid] = tile_byte<MT>(0);      // the zero row
        return;
    }
    for (uint32_t m = 0; m < (uint32_t)MT; m++) {
        if (m >= M) {
            for (uint32_t k = tid; k < d.K; k += nt) dst[(size_t)k * MT + m] = tile_byte<MT>(0);
            continue;
        }
        int amax = 0;
        for (uint32_t k = tid; k < d.K; k += nt) {
            int v = first(A + (size_t)m * d.ldx + k);
            if (B) v += first(B + (size_t)m * d.ldx2 + k);
            amax = max(amax, abs(v));
        }
        amax = __reduce_max_sync(0xffffffffu, amax);
        asm volatile("bar.sync 1, 512;" ::: "memory");       // red[] free to overwrite (consumer warps only)
        if (lane == 0) red[warp] = amax;
        asm volatile("bar.sync 1, 512;" ::: "memory");
        amax = 0;
        for (uint32_t w = 0; w < nwarps; w++) amax = max(amax, red[w]);
        const float scale = amax ? 127.0f / (float)amax : 0.0f;
        for (uint32_t k = tid; k < d.K; k += nt) {
            int v = again(A + (size_t)m * d.ldx + k);
            if (B) v += again(B + (size_t)m * d.ldx2 + k);
            int q = __float2int_rn((float)v * scale);
            q = max(-127, min(127, q));
            dst[(size_t)k * MT + m] = tile_byte<MT>(q);
        }
        if (tid == 0) seq_xscale_s[m] = (float)amax / 127.0f;
        if (write_scale && d.scale_out && tid == 0) d.scale_out[m] = (float)amax / 127.0f;
    }
    if (tid < (uint32_t)MT) dst[(size_t)d.K * MT + tid] = tile_byte<MT>(0);          // the zero row
}

// x_kind 3: the rows' largest magnitudes are already known (recorded by the producing step), so
// one pass over X quantises it: q = clamp(rint(v * (127 / amax)), -127, 127) as in stage_x_quant.
// UNTAG: the source words carry a tag byte to strip (the settled exchange's reader of a few rows).
template <int MT, bool UNTAG = false>
__device__ __forceinline__ void stage_x_scaled(unsigned char *xs, const SeqDesc &d, uint32_t M, const uint32_t *amax, bool write_scale)
{
    [[maybe_unused]] const auto clean = [](int4 v) {
        if constexpr (UNTAG) return make_int4((v.x << 8) >> 8, (v.y << 8) >> 8, (v.z << 8) >> 8, (v.w << 8) >> 8);
        else return v;
    };
    [[maybe_unused]] const auto clean1 = [](int v) { return UNTAG ? (v << 8) >> 8 : v; };
    const uint32_t tid = threadIdx.x, nt = 512;                       // consumer threads only
    float scale[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const uint32_t a = (uint32_t)m < M ? __ldcg(amax + m) : 0u;
        scale[m] = a ? 127.0f / (float)a : 0.0f;
        if (tid == (uint32_t)m) seq_xscale_s[m] = (float)a / 127.0f;
        if (write_scale && d.scale_out && tid == (uint32_t)m && (uint32_t)m < M) d.scale_out[m] = (float)a / 127.0f;
    }
    const bool vec = (d.K & 3) == 0 && (d.ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(d.X) & 15) == 0;
    if constexpr (MT == 1) {
        const int32_t *A = reinterpret_cast<const int32_t *>(d.X);
        if (vec) {
            for (uint32_t q = tid; q < d.K / 4; q += nt) {
                const int4 v = clean(__ldcg(reinterpret_cast<const int4 *>(A) + q));
                const uint32_t w = (uint32_t)(quant1(v.x, scale[0]) & 0xff) | ((uint32_t)(quant1(v.y, scale[0]) & 0xff) << 8) |
                                   ((uint32_t)(quant1(v.z, scale[0]) & 0xff) << 16) | ((uint32_t)(quant1(v.w, scale[0]) & 0xff) << 24);
                reinterpret_cast<uint32_t *>(xs)[q] = w;
            }
        } else {
            for (uint32_t k = tid; k < d.K; k += nt) xs[k] = (unsigned char)quant1(clean1(__ldcg(A + k)), scale[0]);
        }
        if (tid == 0) xs[d.K] = 0;
    } else {
        int8_t *dst = reinterpret_cast<int8_t *>(xs);
        if (vec && MT >= 4) {
            if constexpr (MT >= 4) {
                const int4 *A = reinterpret_cast<const int4 *>(d.X);
                const uint32_t lda = d.ldx / 4;
                const uint32_t quads = d.K / 4, rot = cta_rotation(quads);
                for (uint32_t q0 = tid; q0 < quads; q0 += nt) {
                    const uint32_t q = rotated(q0, rot, quads);
#pragma unroll
                    for (int g = 0; g < MT / 4; g++) {
                        int4 v[4];
#pragma unroll
                        for (int r = 0; r < 4; r++)
                            v[r] = (uint32_t)(4 * g + r) < M ? clean(__ldcg(A + (size_t)(4 * g + r) * lda + q)) : make_int4(0, 0, 0, 0);
                        uint32_t o[4];
#define SPTMM_PACK4(f) ((uint32_t)(quant1(v[0].f, scale[4 * g]) & 0xff) | ((uint32_t)(quant1(v[1].f, scale[4 * g + 1]) & 0xff) << 8) | \
                        ((uint32_t)(quant1(v[2].f, scale[4 * g + 2]) & 0xff) << 16) | ((uint32_t)(quant1(v[3].f, scale[4 * g + 3]) & 0xff) << 24))
                        o[0] = SPTMM_PACK4(x) ^ 0x80808080u;
                        o[1] = SPTMM_PACK4(y) ^ 0x80808080u;
                        o[2] = SPTMM_PACK4(z) ^ 0x80808080u;
                        o[3] = SPTMM_PACK4(w) ^ 0x80808080u;
#undef SPTMM_PACK4
                        if constexpr (MT == 4) {
                            *reinterpret_cast<uint4 *>(xs + (size_t)q * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                *reinterpret_cast<uint32_t *>(xs + ((size_t)q * 4 + i) * MT + 4 * g) = o[i];
                        }
                    }
                }
            }
        } else {
            const int32_t *A = reinterpret_cast<const int32_t *>(d.X);
            for (uint32_t m = 0; m < (uint32_t)MT; m++)
                for (uint32_t k = tid; k < d.K; k += nt)
                    dst[(size_t)k * MT + m] = tile_byte<MT>(m < M ? quant1(clean1(__ldcg(A + (size_t)m * d.ldx + k)), scale[m]) : 0);
        }
        if (tid < (uint32_t)MT) dst[(size_t)d.K * MT + tid] = tile_byte<MT>(0);
    }
}

// int8 rows with a row stride, read around L1 (the buffer may have been written by other CTAs)
template <int MT>
__device__ __forceinline__ void stage_x_i8(unsigned char *xs, const SeqDesc &d, uint32_t M)
{
    const int8_t *X = reinterpret_cast<const int8_t *>(d.X);
    int8_t *dst = reinterpret_cast<int8_t *>(xs);
    const uint32_t tid = threadIdx.x, nt = 512;          // consumer threads only
    if (MT == 1 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) {
        // every CTA starts at a different place: CTAs released together by a step barrier would
        // otherwise all ask the same few L2 lines at the same moment
        const uint32_t vec = d.K / 16, rot = (blockIdx.x * 37u) % max(vec, 1u);
        for (uint32_t i = tid; i < vec; i += nt) {
            const uint32_t j = i + rot < vec ? i + rot : i + rot - vec;
            reinterpret_cast<uint4 *>(xs)[j] = __ldcg(reinterpret_cast<const uint4 *>(X) + j);
        }
        for (uint32_t k = vec * 16 + tid; k < d.K; k += nt) dst[k] = __ldcg(X + k);
    } else if (MT >= 4 && (d.K & 3) == 0 && (d.ldx & 3) == 0 && (reinterpret_cast<uintptr_t>(X) & 3) == 0) {
        // a thread takes four consecutive k from every row (coalesced along k), transposes the
        // 4 x MT bytes in registers and writes four finished tile rows with 16-byte stores
        if constexpr (MT >= 4) {
            const uint32_t quads = d.K / 4;
            for (uint32_t q = tid; q < quads; q += nt) {
                uint32_t w[MT], o[MT];
#pragma unroll
                for (int m = 0; m < MT; m++)
                    w[m] = (uint32_t)m < M ? __ldcg(reinterpret_cast<const uint32_t *>(X + (size_t)m * d.ldx) + q) : 0u;
                transpose_bytes4<MT>(w, o);
                uint4 *out = reinterpret_cast<uint4 *>(xs + (size_t)q * 4 * MT);
#pragma unroll
                for (int i = 0; i < MT / 4; i++)
                    out[i] = make_uint4(o[4 * i] ^ kTileBias<MT>, o[4 * i + 1] ^ kTileBias<MT>,
                                        o[4 * i + 2] ^ kTileBias<MT>, o[4 * i + 3] ^ kTileBias<MT>);
            }
        }
    } else {
        for (uint32_t m = 0; m < (uint32_t)MT; m++)
            for (uint32_t k = tid; k < d.K; k += nt)
                dst[(size_t)k * MT + m] = tile_byte<MT>(m < M ? (int)__ldcg(X + (size_t)m * d.ldx + k) : 0);
    }
    if (tid < (uint32_t)MT) dst[(size_t)d.K * MT + tid] = tile_byte<MT>(0);
}

// x_kind 4: X is the packed int8 copy of a step's output that the producing step made itself.
// Word j*K + k holds rows 3j..3j+2 of column k in its low three bytes and the run's tag in the top
// one (rows past M are zero); a thread takes whole columns, waits until their words carry `tag`
// (bounded), and writes the column's MT tile bytes with one store.
template <int MT>
__device__ __forceinline__ void stage_x_packed(unsigned char *xs, const uint32_t *src, uint32_t K, uint32_t M, uint32_t tag,
                                               bool sys, bool &ok)
{
    constexpr int W3 = (MT + 2) / 3;               // words per column at most
    constexpr int U = MT == 16 ? 2 : 4;            // columns a thread has in flight
    const uint32_t w3 = packed_words(M);
    const uint32_t tid = threadIdx.x, nt = 512;    // consumer threads only
    for (uint32_t k0 = tid; k0 < K; k0 += nt * U) {
        uint32_t w[U][W3];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int j = 0; j < W3; j++) {
                const uint32_t k = k0 + u * nt;
                w[u][j] = (k < K && (uint32_t)j < w3) ? __ldcg(src + (size_t)j * K + k) : 0u;
            }
        for (uint32_t it = 0; ok; it++) {
            bool stale = false;
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int j = 0; j < W3; j++) {
                    const uint32_t k = k0 + u * nt;
                    if (k < K && (uint32_t)j < w3 && (w[u][j] >> 24) != tag) {
                        stale = true;
                        w[u][j] = (uint32_t)ld_fresh(reinterpret_cast<const int32_t *>(src + (size_t)j * K + k), sys);
                    }
                }
            if (!stale) break;
            if (it >= kPollLimit) ok = false;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t k = k0 + u * nt;
            if (k >= K) continue;
            if constexpr (MT == 1) {
                xs[k] = (unsigned char)(w[u][0] & 0xffu);
            } else {
                uint32_t o[MT / 4];
#pragma unroll
                for (int q = 0; q < MT / 4; q++) {
                    o[q] = 0;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int m = 4 * q + i;
                        o[q] |= ((w[u][m / 3] >> (8 * (m % 3))) & 0xffu) << (8 * i);
                    }
                    o[q] ^= 0x80808080u;
                }
                if constexpr (MT == 4) *reinterpret_cast<uint32_t *>(xs + (size_t)k * 4) = o[0];
                else if constexpr (MT == 8) *reinterpret_cast<uint2 *>(xs + (size_t)k * 8) = make_uint2(o[0], o[1]);
                else *reinterpret_cast<uint4 *>(xs + (size_t)k * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
    if (tid < (uint32_t)MT) reinterpret_cast<int8_t *>(xs)[(size_t)K * MT + tid] = tile_byte<MT>(0);      // the zero row
}

constexpr uint32_t kConsumers = 16;          // consumer warps; warp 16 is the producer
constexpr uint32_t kConsumerThreads = kConsumers * 32;

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// One arrival of this CTA at a local counter, then wait until every CTA of this GPU has arrived
// (thread 0 polls, bounded; the others wait at the CTA barrier).  The release covers what the
// CTA's threads wrote before the barrier in front of it.
// BAR / COUNT name the CTA barrier of the threads that take part (the consumers, or the settle warps
// of the pipelined kernel); `leader` is the one thread that arrives and polls.
template <int BAR, int COUNT>
__device__ __forceinline__ void settle_barrier_on(unsigned long long *ctr, unsigned long long target, uint32_t *failed, uint32_t *status,
                                                  uint32_t poll_limit, bool leader)
{
    asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(COUNT) : "memory");
    if (leader) {
        asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(ctr) : "memory");
        if (!*failed) {
            unsigned long long v = 0;
            for (uint32_t it = 0; it < poll_limit; it++) {
                asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
                if (v >= target) break;
            }
            if (v < target) { *failed = 1; atomicOr(status, 16u); }
        }
    }
    asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(COUNT) : "memory");
}
__device__ __forceinline__ void settle_barrier(unsigned long long *ctr, unsigned long long target, uint32_t *failed, uint32_t *status,
                                               uint32_t poll_limit)
{
    settle_barrier_on<1, 512>(ctr, target, failed, status, poll_limit, threadIdx.x == 0);
}

// x_kind 5, the settled exchange.  The producing step stored tagged int32 words (into every rank's
// copy of the buffer, across GPUs).  Having all threads of all CTAs poll those words makes every CTA
// hammer the same few cache lines, which is slow; here every word is watched by exactly ONE CTA of
// each GPU: CTA c owns columns K*c/G .. K*(c+1)/G.  It waits for its columns' words (bounded), and
//  - one row: arrives at a local counter; once all CTAs have, the row is complete in this GPU's L2
//    and every CTA loads and quantises it without further checks;
//  - several rows: adds its columns' row maxima to the step's maxima, arrives; once all have, it
//    quantises ITS columns and writes them as finished tile bytes to a local buffer, arrives at a
//    second counter, and every CTA then takes the whole tile with one bulk copy.
// Only the tagged words cross NVLink; the counters and the tile buffer are local to each GPU.
template <int MT>
__device__ __forceinline__ void stage_x_settled(unsigned char *xs, const SeqDesc &d, const SeqParams &p, uint32_t s, int *red,
                                                uint32_t xbar_a, uint32_t &xphase, uint32_t tag, bool sys, bool &ok,
                                                uint32_t *failed, bool write_scale)
{
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, cta = blockIdx.x, nt = kConsumerThreads;
    const uint32_t k0 = (uint32_t)(((uint64_t)d.K * cta) / p.G), k1 = (uint32_t)(((uint64_t)d.K * (cta + 1)) / p.G), nk = k1 - k0;
    const int32_t *A = reinterpret_cast<const int32_t *>(d.X);
    unsigned long long *c1 = p.settle + 2 * (size_t)s, *c2 = c1 + 1;
    auto arrived = [&](const int32_t *w) {          // wait for one word to carry the tag; returns its value
        int v = __ldcg(w);
        for (uint32_t it = 0; ok && ((uint32_t)v >> 24) != tag; it++) {
            if (it >= p.poll_limit) { ok = false; break; }
            v = ld_fresh(w, sys);
        }
        return untag(v);
    };
    if constexpr (MT == 1) {
        for (uint32_t i = tid; i < nk; i += nt) (void)arrived(A + k0 + i);
        if (!ok && !*failed) { *failed = 1; atomicOr(p.status, 2u); }
        SEQ_MARK(p, s, 0, failed);
        settle_barrier(c1, p.target_local, failed, p.status, p.poll_limit);
        SEQ_MARK(p, s, 1, failed);
        // the row is complete: 16-byte loads, values kept in registers between absmax and rounding
        // (the host admits only rows that fit: K a multiple of 4, at most 14336, 16-byte aligned)
        quant_row_vec(xs, A, d.K, red, true, (write_scale && d.scale_out) ? d.scale_out : nullptr);
        SEQ_MARK(p, s, 2, failed);
    } else {
        int *rowmax_s = red + 32;                          // [16]
        uint32_t *amax_g = p.amax + ((size_t)p.run_parity * p.nsteps + s) * 16;
        unsigned char *tile_g = p.xq + (size_t)(s & 1) * p.xq_stride;
        if (tid < 16) rowmax_s[tid] = 0;
        consumer_sync();
        // thread t owns column k0 + t (a CTA has fewer columns than threads): all rows' loads in flight
        // together, then the stale ones again until they carry the tag
        const bool mine = tid < nk;
        const uint32_t k = k0 + tid;
        int v[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) v[m] = (mine && (uint32_t)m < p.M) ? __ldcg(A + (size_t)m * d.ldx + k) : (int)(tag << 24);
        for (uint32_t it = 0; ok; it++) {
            bool stale = false;
#pragma unroll
            for (int m = 0; m < MT; m++)
                if (((uint32_t)v[m] >> 24) != tag) { stale = true; v[m] = ld_fresh(A + (size_t)m * d.ldx + k, sys); }
            if (!stale) break;
            if (it >= p.poll_limit) ok = false;
        }
        if (warp * 32 < nk) {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                v[m] = untag(v[m]);
                const int a = __reduce_max_sync(0xffffffffu, abs(v[m]));
                if (lane == 0 && a) atomicMax(rowmax_s + m, a);
            }
        }
        if (!ok && !*failed) { *failed = 1; atomicOr(p.status, 2u); }
        consumer_sync();
        SEQ_MARK(p, s, 0, failed);
        if (tid < p.M && rowmax_s[tid]) atomicMax(amax_g + tid, (uint32_t)rowmax_s[tid]);
        settle_barrier(c1, p.target_local, failed, p.status, p.poll_limit);
        SEQ_MARK(p, s, 1, failed);
        float *scale_s = reinterpret_cast<float *>(red);
        if (tid < (uint32_t)MT) {
            const uint32_t a = tid < p.M ? __ldcg(amax_g + tid) : 0u;
            scale_s[tid] = a ? 127.0f / (float)a : 0.0f;
            seq_xscale_s[tid] = (float)a / 127.0f;
            if (write_scale && d.scale_out && tid < p.M) d.scale_out[tid] = (float)a / 127.0f;
        }
        consumer_sync();
        // round my column and put it where the tile has it: bytes k*MT .. k*MT + MT-1, biased, one store
        if (mine) {
            uint32_t o[MT / 4];
#pragma unroll
            for (int q = 0; q < MT / 4; q++) {
                o[q] = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) o[q] |= ((uint32_t)quant1(v[4 * q + i], scale_s[4 * q + i]) & 0xffu) << (8 * i);
                o[q] ^= 0x80808080u;
            }
            if constexpr (MT == 4) *reinterpret_cast<uint32_t *>(tile_g + (size_t)k * 4) = o[0];
            else if constexpr (MT == 8) *reinterpret_cast<uint2 *>(tile_g + (size_t)k * 8) = make_uint2(o[0], o[1]);
            else *reinterpret_cast<uint4 *>(tile_g + (size_t)k * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        settle_barrier(c2, p.target_local, failed, p.status, p.poll_limit);
        SEQ_MARK(p, s, 2, failed);
        // the finished tile: one bulk copy (in pieces of at most 64 KB) into the tile's place
        const uint32_t bytes = d.K * MT;
        if (tid == 0) {
            // the tile bytes were written by other CTAs' ordinary stores, and the tile's place in shared
            // memory was last read by this CTA's gathers: order both before the bulk copy engine's accesses
            asm volatile("fence.proxy.async;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(xbar_a), "r"(bytes) : "memory");
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs);
            for (uint32_t o = 0; o < bytes; o += 65536u) {
                const uint32_t n = min(65536u, bytes - o);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst + o), "l"(tile_g + o), "r"(n), "r"(xbar_a) : "memory");
            }
        }
        if (tid < (uint32_t)MT) xs[(size_t)d.K * MT + tid] = (unsigned char)tile_byte<MT>(0);      // the zero row
        if (!seq_bounded_wait(xbar_a, xphase) && !*failed) { *failed = 1; atomicOr(p.status, 1u); }
        xphase ^= 1;
    }
}

// ---- the pipelined variant of the settled exchange (XV = 3) ------------------------------------
// Two extra warps per CTA (the settle warps) run the whole settle phase of a step -- watch this CTA's
// columns arrive, meet at the local counters, quantise the columns, fetch the finished tile -- into a
// SECOND tile buffer while the sixteen consumer warps are still gathering the step before.  The
// consumers never wait at a counter; they wait for "tile ready" and announce "tile free".  It pays
// when the step list interleaves independent chains (a step's input then comes from the step before
// the previous one and has usually arrived while the previous step is being gathered).
constexpr uint32_t kSettleThreads = 64;
constexpr uint32_t kPipeThreads = kConsumerThreads + 32 + kSettleThreads;

__device__ __forceinline__ void settler_sync() { asm volatile("bar.sync 2, 64;" ::: "memory"); }

// One step's input tile, by the 64 settle threads: `xs` is the tile buffer of this step, `ready_a`
// its "tile ready" barrier.  st = 0..63 numbers the settle threads.
template <int MT>
__device__ __forceinline__ void settle_ahead(unsigned char *xs, uint32_t ready_a, const SeqDesc &d, const SeqParams &p, uint32_t s,
                                             uint32_t st, int *rowmax_s, float *scale_s, float *xscale_out, uint32_t *failed)
{
    static_assert(MT >= 4, "the pipelined exchange is for tiles of several rows");
    const uint32_t cta = blockIdx.x, lane = st & 31;
    const bool sys = p.n_peers != 0;
    if (d.x_kind == 0) {
        // int8 activations as they are: transpose them into the tile (only the first steps of a chain)
        const int8_t *X = reinterpret_cast<const int8_t *>(d.X);
        for (uint32_t i = st; i < d.K * (uint32_t)MT; i += kSettleThreads) {
            const uint32_t k = i / MT, m = i - k * MT;
            xs[i] = (unsigned char)tile_byte<MT>(m < p.M ? (int)__ldcg(X + (size_t)m * d.ldx + k) : 0);
        }
        if (st < (uint32_t)MT) xs[(size_t)d.K * MT + st] = (unsigned char)tile_byte<MT>(0);      // the zero row
        if (st < 16) xscale_out[st] = 1.0f;
        settler_sync();
        if (st == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready_a) : "memory");
        return;
    }
    const uint32_t tag = seq_tag(p.run_mod, d.in_tag_m, d.in_tag_j);
    const uint32_t k0 = (uint32_t)(((uint64_t)d.K * cta) / p.G), k1 = (uint32_t)(((uint64_t)d.K * (cta + 1)) / p.G), nk = k1 - k0;
    const int32_t *A = reinterpret_cast<const int32_t *>(d.X);
    unsigned long long *c1 = p.settle + 2 * (size_t)s, *c2 = c1 + 1;
    uint32_t *amax_g = p.amax + ((size_t)p.run_parity * p.nsteps + s) * 16;
    unsigned char *tile_g = p.xq + (size_t)(s & 1) * p.xq_stride;
    bool ok = *failed == 0;
    if (st < 16) rowmax_s[st] = 0;
    settler_sync();
    // my columns: st, st + 64, ...; the first one's values stay in registers
    int v[MT], am[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) { v[m] = 0; am[m] = 0; }
    for (uint32_t c = st; c < nk; c += kSettleThreads) {
        const uint32_t k = k0 + c;
        int w[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) w[m] = (uint32_t)m < p.M ? __ldcg(A + (size_t)m * d.ldx + k) : (int)(tag << 24);
        for (uint32_t it = 0; ok; it++) {
            bool stale = false;
#pragma unroll
            for (int m = 0; m < MT; m++)
                if (((uint32_t)w[m] >> 24) != tag) { stale = true; w[m] = ld_fresh(A + (size_t)m * d.ldx + k, sys); }
            if (!stale) break;
            if (it >= p.poll_limit) ok = false;
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            w[m] = untag(w[m]);
            am[m] = max(am[m], abs(w[m]));
            if (c == st) v[m] = w[m];
        }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const int a = __reduce_max_sync(0xffffffffu, am[m]);
        if (lane == 0 && a) atomicMax(rowmax_s + m, a);
    }
    if (!ok && !*failed) { *failed = 1; atomicOr(p.status, 2u); }
    settler_sync();
    SEQ_MARK_BY(p, s, 0, failed, kConsumerThreads + 33);
    if (st < p.M && rowmax_s[st]) atomicMax(amax_g + st, (uint32_t)rowmax_s[st]);
    settle_barrier_on<2, 64>(c1, p.target_local, failed, p.status, p.poll_limit, st == 0);
    SEQ_MARK_BY(p, s, 1, failed, kConsumerThreads + 33);
    if (st < (uint32_t)MT) {
        const uint32_t a = st < p.M ? __ldcg(amax_g + st) : 0u;
        scale_s[st] = a ? 127.0f / (float)a : 0.0f;
        xscale_out[st] = (float)a / 127.0f;
        if (cta == 0 && d.scale_out && st < p.M) d.scale_out[st] = (float)a / 127.0f;
    }
    settler_sync();
    for (uint32_t c = st; c < nk; c += kSettleThreads) {
        const uint32_t k = k0 + c;
        uint32_t o[MT / 4];
#pragma unroll
        for (int q = 0; q < MT / 4; q++) {
            o[q] = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int m = 4 * q + i;
                const int val = c == st ? v[m] : ((uint32_t)m < p.M ? untag(__ldcg(A + (size_t)m * d.ldx + k)) : 0);
                o[q] |= ((uint32_t)quant1(val, scale_s[m]) & 0xffu) << (8 * i);
            }
            o[q] ^= 0x80808080u;
        }
        if constexpr (MT == 4) *reinterpret_cast<uint32_t *>(tile_g + (size_t)k * 4) = o[0];
        else if constexpr (MT == 8) *reinterpret_cast<uint2 *>(tile_g + (size_t)k * 8) = make_uint2(o[0], o[1]);
        else *reinterpret_cast<uint4 *>(tile_g + (size_t)k * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    settle_barrier_on<2, 64>(c2, p.target_local, failed, p.status, p.poll_limit, st == 0);
    SEQ_MARK_BY(p, s, 2, failed, kConsumerThreads + 33);
    if (st < (uint32_t)MT) xs[(size_t)d.K * MT + st] = (unsigned char)tile_byte<MT>(0);      // the zero row
    settler_sync();
    if (st == 0) {
        const uint32_t bytes = d.K * MT;
        asm volatile("fence.proxy.async;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ready_a), "r"(bytes) : "memory");
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs);
        for (uint32_t o = 0; o < bytes; o += 65536u) {
            const uint32_t n = min(65536u, bytes - o);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dst + o), "l"(tile_g + o), "r"(n), "r"(ready_a) : "memory");
        }
    }
}

// XV selects what a kernel variant knows about (each carries only its own code, which keeps the
// registers of the input stages it does not need out of the gather loop's way):
//   0  int8 inputs and the counter hand-over (x_kind 0, 1)
//   1  also tagged words polled by every reader, row maxima, the producer-side quantiser (x_kind 2, 3, 4)
//   2  int8 inputs and the settled exchange (x_kind 0, 5)
//   3  the same with the settle phase in two warps of its own, one step ahead of the gather (see settle_ahead)
template <int MT, int XV>
__global__ void __launch_bounds__(XV == 3 ? kPipeThreads : kConsumerThreads + 32, 1) k_seq(const __grid_constant__ SeqParams p)
{
    constexpr bool TAGGED = XV == 1;          // the polling exchanges
    constexpr bool SETTLED = XV == 2;
    constexpr bool PIPE = XV == 3;
    constexpr bool TAGS = XV != 0;            // outputs may carry tags
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    unsigned char *smem = tile_base(dyn_smem);     // the tile's fixed address; all offsets count from it
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, R = p.ring_slots;
    const uint32_t slot_blocks = p.slot_blocks, slot_bytes = slot_blocks * 512;
    const bool producer = warp == kConsumers;

    // ---- shared memory: X tile (two of them in the pipelined variant) | column sums (two buffers) | scratch | barriers | rings
    unsigned char *xs = smem;
    const size_t tiles_bytes = PIPE ? 2 * (size_t)p.xs_bytes : (size_t)p.xs_bytes;
    int *c_base = reinterpret_cast<int *>(smem + tiles_bytes);
    int *red = c_base + 2 * (size_t)p.max_cols * MT;
    size_t o = tiles_bytes + (2 * (size_t)p.max_cols * MT + kRedInts) * 4;
    o = (o + 7) & ~(size_t)7;
    const uint32_t bars_a = (uint32_t)__cvta_generic_to_shared(smem + o);     // [warp][full R | empty R]
    o += (size_t)kConsumers * 2 * R * 8;
    o = (o + 127) & ~(size_t)127;
    unsigned char *rings = smem + o;                                           // [warp][R][slot_bytes]
    __shared__ uint32_t failed;              // a bounded wait ran out somewhere in this CTA
    __shared__ __align__(16) uint32_t desc_s[2][(sizeof(SeqDesc) + 15) / 16 * 4];   // this and the next step's descriptor
    __shared__ uint32_t meta_s[2][4];        // their plan entries: b0, b1, c0, c1
    __shared__ float xscale_keep[2][16];     // the input rows' scales of this and the previous step (c_kind 2)
    __shared__ __align__(8) unsigned long long xbar;        // completion of the activation tile's bulk copy (x_kind 5)
    const uint32_t xbar_a = (uint32_t)__cvta_generic_to_shared(&xbar);
    uint32_t xphase = 0;
    // pipelined variant: per tile buffer, "ready" (filled by the settle warps) and "free" (gathered by the consumers)
    __shared__ __align__(8) unsigned long long tile_bar[4];
    __shared__ float xscale_buf[2][16];
    __shared__ int settle_rowmax_s[16];
    __shared__ float settle_scale_s[16];
    const uint32_t ready_a = (uint32_t)__cvta_generic_to_shared(&tile_bar[0]), free_a = ready_a + 16;
    if (tid == 0) {
        failed = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(xbar_a) : "memory");
        if constexpr (PIPE)
            for (uint32_t i = 0; i < 4; i++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(ready_a + 8 * i) : "memory");
    }
    if (warp < kConsumers && lane == 0) {
        for (uint32_t i = 0; i < 2 * R; i++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bars_a + (warp * 2 * R + i) * 8) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // ================= producer warp: lane w keeps consumer warp w's ring full =================
    if (producer) {
        if (lane >= kConsumers) return;
        const uint32_t w = lane;
        const uint32_t full_a = bars_a + w * 2 * R * 8, empty_a = full_a + R * 8;
        const uint32_t ring_a = (uint32_t)__cvta_generic_to_shared(rings + (size_t)w * R * slot_bytes);
        // Lock-step state machine: the 16 lanes poll and issue together, so one instruction of
        // this warp moves up to 16 rings forward (diverged lanes would serialise ~50 copies a step).
        uint32_t slot = 0, par = 1;          // parity 1 on a fresh barrier passes: all slots start empty
        uint32_t s = 0xffffffffu, pb = 0, pend = 0, spins = 0;
        const uint4 *idx = nullptr;
        bool done = false;
        while (true) {
            if (!done && pb >= pend) {       // move to the next step (one per iteration; empty slices just pass)
                if (++s >= p.nsteps) done = true;
                else {
                    const uint32_t b0 = __ldg(p.cta_blk + (size_t)s * (p.G + 1) + cta);
                    const uint32_t b1 = __ldg(p.cta_blk + (size_t)s * (p.G + 1) + cta + 1);
                    idx = p.desc[s].idx;
                    const uint32_t nb = b1 - b0;
                    pb = b0 + (uint32_t)(((uint64_t)nb * w) / kConsumers);
                    pend = b0 + (uint32_t)(((uint64_t)nb * (w + 1)) / kConsumers);
                }
            }
            if (!done && pb < pend) {
                uint32_t ready;
                asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                             : "=r"(ready) : "r"(empty_a + slot * 8), "r"(par) : "memory");
                if (ready) {
                    const uint32_t cnt = min(slot_blocks, pend - pb);
                    seq_bulk_fetch(ring_a + slot * slot_bytes, idx + (size_t)pb * 32, cnt * 512u, full_a + slot * 8);
                    pb += cnt;
                    if (++slot == R) { slot = 0; par ^= 1; }
                    spins = 0;
                } else if (++spins > (1u << 26)) {      // the consumer never freed the slot: report, stop
                    atomicOr(p.status, 4u);
                    done = true;
                }
            }
            if (__all_sync(0x0000ffffu, done)) break;
        }
        return;
    }

    // ================= settle warps (pipelined variant): one step ahead of the consumers =================
    if constexpr (PIPE) {
        if (warp > kConsumers) {
            const uint32_t st = tid - (kConsumerThreads + 32);
            uint32_t free_phase[2] = {0, 0};
            for (uint32_t t = 0; t < p.nsteps; t++) {
                const uint32_t b = t & 1;
                if (t >= 2) {            // the buffer's previous tile must have been gathered
                    // (after a failure nothing waits any more: the consumers stop waiting for their tiles
                    // too, so the two sides' phases no longer line up and a wait here would only run out)
                    if (!failed && !seq_bounded_wait(free_a + 8 * b, free_phase[b])) { failed = 1; atomicOr(p.status, 4u); }
                    free_phase[b] ^= 1;
                }
                settle_ahead<MT>(xs + (size_t)b * p.xs_bytes, ready_a + 8 * b, p.desc[t], p, t, st, settle_rowmax_s, settle_scale_s,
                                 xscale_buf[b], &failed);
            }
            return;
        }
    }

    // ================= consumer warps =================
    // the first threads carry one word each of a step's descriptor, threads 64..67 its plan entries
    static_assert(sizeof(SeqDesc) % 4 == 0 && sizeof(SeqDesc) / 4 <= 64, "a descriptor travels in the first 64 threads");
    auto load_step_word = [&](uint32_t st) -> uint32_t {
        if (tid < sizeof(SeqDesc) / 4) return __ldg(reinterpret_cast<const uint32_t *>(p.desc + st) + tid);
        if (tid >= 64 && tid < 68) {
            const uint32_t *row = (tid < 66 ? p.cta_blk : p.cta_col) + (size_t)st * (p.G + 1) + cta;
            return __ldg(row + (tid & 1));
        }
        return 0;
    };
    auto store_step_word = [&](uint32_t st, uint32_t v) {
        if (tid < sizeof(SeqDesc) / 4) desc_s[st & 1][tid] = v;
        if (tid >= 64 && tid < 68) meta_s[st & 1][tid - 64] = v;
    };
    store_step_word(0, load_step_word(0));
    consumer_sync();
    const uint32_t full_a = bars_a + warp * 2 * R * 8, empty_a = full_a + R * 8;
    const uint32_t ring_sa = (uint32_t)__cvta_generic_to_shared(rings + (size_t)warp * R * slot_bytes) + lane * 16;
    uint32_t cslot = 0, cpar = 0;            // consumer cursor: slot and phase parity
    [[maybe_unused]] uint32_t ready_phase[2] = {0, 0};
    int held_slot = -1;                      // a consumed slot whose release is deferred (see below)
    bool ring_ok = true;

    for (uint32_t s = 0; s < p.nsteps; s++) {
        // descriptor and plan entries of this step: put in shared memory during the previous step
        // (read in place: a private copy of the descriptor would live in local memory)
        const SeqDesc &d = *reinterpret_cast<const SeqDesc *>(desc_s[s & 1]);
        const uint32_t b0 = meta_s[s & 1][0], b1 = meta_s[s & 1][1], c0 = meta_s[s & 1][2], c1 = meta_s[s & 1][3];
        int *c_s = c_base + (s & 1) * (size_t)p.max_cols * MT;
#ifdef SPTMM_TUNING
        const bool tracing = p.trace != nullptr && cta == 0 && tid == 33 && s < 256;
#endif
        // ---- wait until the step this one depends on has finished everywhere
        if (d.dep >= 0 && !(TAGGED && (d.x_kind == 2 || d.x_kind == 4)) && !((SETTLED || PIPE) && d.x_kind == 5)) {     // tagged inputs are waited for word by word while staging
            if (tid == 0 && !failed) {
                const unsigned long long *ctr = p.counters + d.dep;
                unsigned long long v = 0;
                for (uint32_t it = 0; it < p.poll_limit; it++) {
                    if (p.n_peers) asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
                    else asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ctr) : "memory");
                    if (v >= p.target) break;
                }
                if (v < p.target) { failed = 1; atomicOr(p.status, 2u); }
            }
            consumer_sync();
        }
#ifdef SPTMM_TUNING
        if (tracing) p.trace[s * 4 + 0] = seq_ns(&failed);
        if (p.trace != nullptr && cta == 0 && lane == 1 && s >= 100 && s < 104)
            p.trace[1024 + 64 + (s - 100) * 16 + warp] = seq_ns(&failed);
        if (p.trace != nullptr && tid == 33 && s >= 100 && s < 104) p.trace[2048 + (s - 100) * 256 + cta] = seq_ns(&failed);   // every CTA: past the wait
#endif

        // ---- activations and column sums
        const uint32_t ncols = c1 - c0;
        // ask for the next step's descriptor and plan entries now; they are stored after the loop,
        // so their latency (long right after a step barrier, when every CTA asks the same few
        // L2 lines) hides behind the gathers
        uint32_t nxt = 0;
        if (s + 1 < p.nsteps) nxt = load_step_word(s + 1);
        // (TAGGED kernels are the ones that also know row maxima: plain sequences carry neither)
        if (TAGS && p.amax != nullptr && cta == 0 && tid < 16)        // the other half of the row maxima: clean for the next run
            p.amax[((p.run_parity ^ 1u) * p.nsteps + s) * 16 + tid] = 0u;
        [[maybe_unused]] const uint32_t xoff = PIPE ? (s & 1) * p.xs_bytes : 0u;      // which tile buffer this step gathers from
        if constexpr (PIPE) {
            // the settle warps fill this step's tile (int8 inputs too); wait for it
            if (!failed && !seq_bounded_wait(ready_a + 8 * (s & 1), ready_phase[s & 1])) { failed = 1; atomicOr(p.status, 1u); }
            ready_phase[s & 1] ^= 1;
            if (tid < 16) seq_xscale_s[tid] = xscale_buf[s & 1][tid];
        }
        else if (d.x_kind == 0) {
            stage_x_i8<MT>(xs, d, p.M);
            if (tid < 16) seq_xscale_s[tid] = 1.0f;          // int8 activations come as they are
        }
        else if constexpr (SETTLED) {               // x_kind 5 (the host admits no other kind here)
            bool fresh = failed == 0;
            const uint32_t tag = seq_tag(p.run_mod, d.in_tag_m, d.in_tag_j);
            stage_x_settled<MT>(xs, d, p, s, red, xbar_a, xphase, tag, p.n_peers != 0, fresh, &failed, cta == 0);
            if (!fresh && !failed) { failed = 1; atomicOr(p.status, 2u); }
        }
        else if (TAGGED && d.x_kind == 4) {
            bool fresh = failed == 0;
            stage_x_packed<MT>(xs, reinterpret_cast<const uint32_t *>(d.X), d.K, p.M, 1u + p.run_mod, p.n_peers != 0, fresh);
            if (!fresh && !failed) { failed = 1; atomicOr(p.status, 2u); }
        }
        else if (TAGGED && d.x_kind == 3) stage_x_scaled<MT>(xs, d, p.M, p.amax + ((size_t)p.run_parity * p.nsteps + (uint32_t)d.dep) * 16, cta == 0);
        else {
            bool fresh = failed == 0;          // after a failure nothing waits any more
            const uint32_t tag = (TAGGED && d.x_kind == 2) ? seq_tag(p.run_mod, d.in_tag_m, d.in_tag_j) : 0u;
            stage_x_quant<MT, TAGGED>(xs, d, p.M, red, cta == 0, tag, p.n_peers != 0, fresh);
            if (!fresh && !failed) { failed = 1; atomicOr(p.status, 2u); }      // a producer's word never arrived
        }
#ifdef SPTMM_TUNING
        if (p.trace != nullptr && cta == 0 && lane == 1 && s >= 100 && s < 104)
            p.trace[1024 + (s - 100) * 16 + warp] = seq_ns(&failed) + (xs[tid] == 77 && xs[tid + 1] == 78 && xs[tid + 2] == 99);
#endif
        for (uint32_t i = tid; i < ncols * MT; i += kConsumerThreads) c_s[i] = 0;
        consumer_sync();
        // the rows' scales, kept per step parity: the next step's input stage overwrites seq_xscale_s
        // while slow threads may still be storing this step's results
        if (tid < 16) xscale_keep[s & 1][tid] = seq_xscale_s[tid];
        if (held_slot >= 0) {                  // X is in: now the previous step's last slot may refill
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_a + held_slot * 8) : "memory");
            held_slot = -1;
        }
#ifdef SPTMM_TUNING
        if (tracing) p.trace[s * 4 + 1] = seq_ns(&failed);
        if (p.trace != nullptr && tid == 33 && s >= 100 && s < 104) p.trace[3072 + (s - 100) * 256 + cta] = seq_ns(&failed);   // every CTA: X staged
#endif

        // ---- gather this warp's blocks out of its ring
        const uint32_t nb = b1 - b0;
        const uint32_t wb0 = b0 + (uint32_t)(((uint64_t)nb * warp) / kConsumers);
        const uint32_t wb1 = b0 + (uint32_t)(((uint64_t)nb * (warp + 1)) / kConsumers);
        if (wb0 < wb1) {
            const uint32_t nbl = d.uniform_nbl;
            uint32_t li, bound;
            if (nbl) {
                li = wb0 / nbl - 2 * c0;
                bound = (wb0 / nbl + 1) * nbl;
            } else {
                // lists are few per CTA: count boundaries at or below wb0 straight from global
                li = 0;
                const uint32_t nlists = 2 * ncols;
                for (uint32_t r = 1; r <= nlists; r += 32) {
                    const uint32_t i = r + lane;
                    const uint32_t ov = i <= nlists ? __ldg(d.blk_off + 2 * (size_t)c0 + i) : 0xffffffffu;
                    li += __popc(__ballot_sync(0xffffffffu, ov <= wb0));
                }
                bound = __ldg(d.blk_off + 2 * (size_t)c0 + li + 1);
            }
            LaneAcc<SPTMM_I8, MT> acc;
            acc.clear(p.one, xoff);
            bool dirty = false;
            PendingSums<MT> done;
            done.clear();
            auto flush = [&]() {
                acc.finish();
                done.push(acc.v, li >> 1, (li & 1) != 0, c_s, lane);
            };
            auto gather8 = [&](const uint4 v) {
                acc.reserve(8);
                acc.add(v.x & 0xffffu);
                acc.add(v.x >> 16);
                acc.add(v.y & 0xffffu);
                acc.add(v.y >> 16);
                acc.add(v.z & 0xffffu);
                acc.add(v.z >> 16);
                acc.add(v.w & 0xffffu);
                acc.add(v.w >> 16);
            };
#ifdef SPTMM_TUNING
            // per-warp view of the gather (two CTAs, steps 100..103): start, time spent waiting for ring slots, slots
            const bool wtr = p.trace != nullptr && lane == 0 && s >= 100 && s < 104 && (cta == 0 || cta == 100);
            unsigned long long w_t0 = wtr ? seq_ns(&failed) : 0ull, w_wait = 0ull;
            uint32_t w_slots = 0;
#endif
            // two blocks of one list at a time: sixteen independent gathers in flight per lane
            auto gather16 = [&](const uint4 v0, const uint4 v1) {
                acc.reserve(16);
                acc.add(v0.x & 0xffffu); acc.add(v1.x & 0xffffu);
                acc.add(v0.x >> 16);     acc.add(v1.x >> 16);
                acc.add(v0.y & 0xffffu); acc.add(v1.y & 0xffffu);
                acc.add(v0.y >> 16);     acc.add(v1.y >> 16);
                acc.add(v0.z & 0xffffu); acc.add(v1.z & 0xffffu);
                acc.add(v0.z >> 16);     acc.add(v1.z >> 16);
                acc.add(v0.w & 0xffffu); acc.add(v1.w & 0xffffu);
                acc.add(v0.w >> 16);     acc.add(v1.w >> 16);
            };
            for (uint32_t b = wb0; b < wb1;) {
                const uint32_t cnt = min(slot_blocks, wb1 - b);
#ifdef SPTMM_TUNING
                const unsigned long long w_ta = wtr ? seq_ns(&failed) : 0ull;
#endif
                if (ring_ok) ring_ok = seq_bounded_wait(full_a + cslot * 8, cpar);
                if (!ring_ok) break;
#ifdef SPTMM_TUNING
                if (wtr) { w_wait += seq_ns(&failed) - w_ta; w_slots++; }
#endif
                const uint32_t slot_a = ring_sa + cslot * slot_bytes;           // this lane's vector of the slot's first block
                // runs of blocks that stay inside one list go through a loop with no checks in it
                for (uint32_t i = 0; i < cnt;) {
                    if (b + i >= bound) {
                        do {
                            if (dirty) { flush(); dirty = false; }
                            li++;
                            bound = nbl ? bound + nbl : __ldg(d.blk_off + 2 * (size_t)c0 + li + 1);
                        } while (b + i >= bound);
                    }
                    const uint32_t run = min(cnt - i, bound - (b + i));
                    uint32_t a = slot_a + i * 512u, j = 0;
                    for (; j + 2 <= run; j += 2, a += 1024u) gather16(lds_vec(a), lds_vec(a + 512u));
                    if (j < run) gather8(lds_vec(a));
                    dirty = true;
                    i += run;
                }
                b += cnt;
                __syncwarp();                  // every lane has the slot's data in registers
                // Free the slot for refilling -- except the step's last one, which is handed back only
                // after the next step's X is staged: its refill would otherwise be in flight to
                // this SM exactly when the latency-critical X loads are.
                if (b < wb1) {
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_a + cslot * 8) : "memory");
                } else {
                    held_slot = (int)cslot;
                }
                if (++cslot == R) { cslot = 0; cpar ^= 1; }
            }
            if (!ring_ok && lane == 0) { failed = 1; atomicOr(p.status, 1u); }
            if (dirty) flush();
            done.drain(c_s, lane);
#ifdef SPTMM_TUNING
            if (wtr) {
                unsigned long long *o = p.trace + 8192 + ((((cta != 0) * 4u + (s - 100)) * 16u + warp) * 4u);
                o[0] = w_t0; o[1] = w_wait; o[2] = seq_ns(&failed); o[3] = w_slots;
            }
#endif
        }
        if (s + 1 < p.nsteps) store_step_word(s + 1, nxt);
        consumer_sync();
        if constexpr (PIPE) {            // this step's tile is gathered: its buffer may take the tile after next
            if (tid == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(free_a + 8 * (s & 1)) : "memory");
        }
#ifdef SPTMM_TUNING
        if (tracing) p.trace[s * 4 + 2] = seq_ns(&failed);
        if (p.trace != nullptr && tid == 33 && s >= 100 && s < 104) p.trace[4096 + (s - 100) * 256 + cta] = seq_ns(&failed);   // every CTA: gathered
#endif

        // what goes out: every column's sum, or (c_kind 1) the sums of neighbouring column pairs;
        // the plan gives a pair-summing step even column boundaries
        const bool pairs = d.c_kind == 1;
        const uint32_t nout = pairs ? ncols / 2 : ncols, o0 = pairs ? c0 / 2 : c0;
        auto value = [&](uint32_t j, uint32_t m) { return pairs ? c_s[(2 * j) * MT + m] + c_s[(2 * j + 1) * MT + m] : c_s[j * MT + m]; };

        // ---- producer-side quantiser (see SeqDesc::q_n): two hand-overs, all consumer warps
        if (TAGGED && d.q_n) {
            const uint32_t qtag = (1u + p.run_mod) << 24;
            const uint32_t ranks = p.n_peers ? p.n_peers : 1u;
            auto area = [&](uint32_t r) { return reinterpret_cast<unsigned char *>(p.n_peers ? p.counter_peers[r] : p.counters); };
            unsigned char *own = reinterpret_cast<unsigned char *>(p.counters);
            // own output columns inside the range, in this step's local column numbers
            const int lo = max((int)o0, d.q_0), hi = min((int)(o0 + nout), d.q_0 + (int)d.q_n);
            float *scale_s = reinterpret_cast<float *>(red);
            if (warp < p.M) {                  // warp r looks after row r
                uint32_t mx = 0;
                for (int c = lo + (int)lane; c < hi; c += 32) mx = max(mx, (uint32_t)abs(value((uint32_t)c - o0, warp)));
                mx = __reduce_max_sync(0xffffffffu, mx);
                // every CTA's maximum of the row, as a tagged word of its own: no counter, no fence
                uint32_t *amax1 = reinterpret_cast<uint32_t *>(own + d.amax1_off) + warp * kAmaxStride;
                if (lane == 0) asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(amax1 + cta), "r"(qtag | mx) : "memory");
                bool okq = failed == 0;
                uint32_t g = 0;
                for (uint32_t c = lane; c < p.G; c += 32) {
                    uint32_t v = (uint32_t)ld_fresh(reinterpret_cast<const int32_t *>(amax1 + c), false);
                    for (uint32_t it = 0; okq && (v & 0xff000000u) != qtag; it++) {
                        if (it >= kPollLimit) { okq = false; break; }
                        v = (uint32_t)ld_fresh(reinterpret_cast<const int32_t *>(amax1 + c), false);
                    }
                    g = max(g, v & 0xffffffu);
                }
                g = __reduce_max_sync(0xffffffffu, g);
                if (p.n_peers > 1) {
                    // between GPUs: CTA r of every rank tells rank r this GPU's maxima; everybody then reads its
                    // own rank's table of the n_peers GPUs' values
                    if (cta < p.n_peers && lane == 0) {
                        uint32_t *dst = reinterpret_cast<uint32_t *>(area(cta) + d.amax2_off) + warp * kMaxPeers + p.my_rank;
                        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(qtag | g) : "memory");
                    }
                    const uint32_t *amax2 = reinterpret_cast<const uint32_t *>(own + d.amax2_off) + warp * kMaxPeers;
                    uint32_t v = qtag;
                    if (lane < p.n_peers) {
                        v = (uint32_t)ld_fresh(reinterpret_cast<const int32_t *>(amax2 + lane), true);
                        for (uint32_t it = 0; okq && (v & 0xff000000u) != qtag; it++) {
                            if (it >= kPollLimit) { okq = false; break; }
                            v = (uint32_t)ld_fresh(reinterpret_cast<const int32_t *>(amax2 + lane), true);
                        }
                    }
                    g = __reduce_max_sync(0xffffffffu, v & 0xffffffu);
                }
                if (!__all_sync(0xffffffffu, okq) && lane == 0 && !failed) { failed = 1; atomicOr(p.status, 8u); }
                if (lane == 0) {
                    scale_s[warp] = g ? 127.0f / (float)g : 0.0f;
                    if (cta == 0 && d.q_scale_out) d.q_scale_out[warp] = (float)g / 127.0f;
                }
            }
            consumer_sync();
            // round this CTA's columns and hand them to every rank: three rows and the tag per word
            const uint32_t w3 = packed_words(p.M);
            const uint32_t nq = hi > lo ? (uint32_t)(hi - lo) : 0u;
            for (uint32_t i = tid; i < nq * w3; i += kConsumerThreads) {
                const uint32_t j = i / nq, c = (uint32_t)lo + (i - j * nq);
                uint32_t word = qtag;
#pragma unroll
                for (uint32_t t = 0; t < 3; t++) {
                    const uint32_t m = 3 * j + t;
                    if (m < p.M) word |= ((uint32_t)quant1(value(c - o0, m), scale_s[m]) & 0xffu) << (8 * t);
                }
                const size_t at = (size_t)j * d.q_n + (uint32_t)((int)c - d.q_0);
                for (uint32_t r = 0; r < ranks; r++) {
                    uint32_t *dst = reinterpret_cast<uint32_t *>(area(r) + d.q_off) + at;
                    if (p.n_peers) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(word) : "memory");
                    else asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(dst), "r"(word) : "memory");
                }
            }
        }

        // ---- results out, then tell the other CTAs this step is done here.  A handful of values
        // that a counter bump has to follow are stored by warp 0 alone while the others move on (the
        // next step accumulates into the other buffer); otherwise all warps store.
        // A tagged output carries its tag in the top byte (|value| < 2^23 because K < 65536).
        const bool tag_out = TAGS && d.out_tag_m != 0;
        const uint32_t otag = tag_out ? seq_tag(p.run_mod, d.out_tag_m, d.out_tag_j) << 24 : 0u;
        const bool tail = (TAGGED && d.want_amax) || d.release;      // something follows the stores
        const bool solo = tail && nout * p.M <= 64;
        auto store_out = [&](uint32_t first, uint32_t step) {
            for (uint32_t i = first; i < nout * p.M; i += step) {
                const uint32_t m = i / nout, j = i - m * nout;
                const int val = value(j, m);
                // c_kind 2: the de-quantised result, float(sum) * (absmax / 127 of the input row), stored as a float
                const int wv = d.c_kind == 2 ? __float_as_int((float)val * xscale_keep[s & 1][m])
                                             : (tag_out ? (int)(otag | ((uint32_t)val & 0xffffffu)) : val);
                if (p.n_peers == 0) d.C[(size_t)m * d.ldc + o0 + j] = wv;
                else                  // the exchange: straight into every rank's buffer over NVLink (plain peer stores)
                    for (uint32_t r = 0; r < p.n_peers; r++) d.Cp[r][(size_t)m * d.ldc + o0 + j] = wv;
            }
        };
        if (!solo) {
            store_out(tid, kConsumerThreads);
            if (tail) consumer_sync();
        }
        if (warp == 0 && (solo || tail)) {
            if (solo) store_out(lane, 32);
            if (TAGGED && d.want_amax) {        // every row's largest magnitude, for the x_kind 3 reader: lane m reports row m
                uint32_t mine = 0;
                for (uint32_t m = 0; m < p.M; m++) {
                    uint32_t mx = 0;
                    for (uint32_t j = lane; j < nout; j += 32) mx = max(mx, (uint32_t)abs(value(j, m)));
                    mx = __reduce_max_sync(0xffffffffu, mx);
                    if (lane == m) mine = mx;
                }
                const size_t slot = ((size_t)p.run_parity * p.nsteps + s) * 16 + lane;
                if (lane < p.M) {
                    if (p.n_peers == 0) atomicMax(p.amax + slot, mine);
                    else
                        for (uint32_t r = 0; r < p.n_peers; r++) atomicMax_system(p.amax_peers[r] + slot, mine);
                }
            }
            __syncwarp();
            // the release orders this warp's stores and reductions (seen through __syncwarp) before the count
            if (p.n_peers == 0) {
                if (lane == 0 && d.release) asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(p.counters + s) : "memory");
            } else if (lane < p.n_peers && d.release) {
                asm volatile("red.release.sys.global.add.u64 [%0], 1;" ::"l"(p.counter_peers[lane] + s) : "memory");
            }
        }
#ifdef SPTMM_TUNING
        if (tracing) p.trace[s * 4 + 3] = seq_ns(&failed);
#endif
    }
}

}  // namespace sptmm

// ---------------------------------------------------------------------------------------------
using namespace sptmm;

struct sptmm_seq {
    int device = -1;
    uint32_t nsteps = 0, M = 0, mt = 0, G = 0, threads = 544, max_cols = 1, ring_slots = 0, xs_bytes = 0, slot_blocks = 8;
    size_t smem = 0;
    uint64_t stream_bytes = 0;       // encoded bytes one run reads
    uint64_t epoch = 0;
    void *d_desc = nullptr, *d_blk = nullptr, *d_col = nullptr, *d_counters = nullptr, *d_status = nullptr;
    void *d_trace = nullptr;
    void *d_xq = nullptr;            // x_kind 5: two local buffers for the finished int8 tile
    uint32_t xq_stride = 0;
    uint32_t n_peers = 0, my_rank = 0;
    bool tagged = false;             // some step reads tagged words: run the kernel variant that knows them
    bool uses_amax = false;          // some step is x_kind 3: the row-maxima area is in use
    bool settled = false;            // the steps with a producer are all x_kind 5: the kernel variant for that exchange
    bool pipe = false;               // ... with the settle phase in warps of its own, one step ahead
    uint32_t poll_limit = 1u << 21;  // see sptmm_seq_set_wait_limit
    void *counter_peers[kMaxPeers] = {};
};

// Shallow rings stream best: three 4 KB slots per warp reach the HBM rate, deeper ones lose it.
static size_t seq_ring_cap()
{
    return (size_t)std::max(2L, std::min(tuning_knob("SPTMM_SEQ_RING", 3), 24L));
}

static void seq_release(sptmm_seq *q)
{
    if (!q) return;
    if (q->device >= 0) {
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(q->device);
        for (void *p : {q->d_desc, q->d_blk, q->d_col, q->d_counters, q->d_status, q->d_xq}) if (p) cudaFree(p);
        cudaSetDevice(cur);
    }
    delete q;
}

// The synchronisation area of one rank: step counters (n x u64), the row maxima of x_kind 3
// (2 halves x n steps x 16 rows x u32), then, for every step that quantises its own output for an
// x_kind 4 reader, its tables of row maxima and its packed int8 output.  The same on every rank.
struct SeqLayout {
    std::vector<uint32_t> q_n, q_off, amax1_off, amax2_off;     // per producing step (q_n == 0: none)
    uint64_t bytes = 0;
};

static SeqLayout seq_layout(const sptmm_seq_step *steps, uint32_t n, uint32_t M)
{
    SeqLayout L;
    L.q_n.assign(n, 0); L.q_off.assign(n, 0); L.amax1_off.assign(n, 0); L.amax2_off.assign(n, 0);
    uint64_t at = (uint64_t)n * 8 + (uint64_t)2 * n * 16 * 4 + (uint64_t)n * 16;      // = sptmm_seq_shared_bytes(n)
    for (uint32_t s = 0; s < n; s++)
        if (steps[s].x_kind == 4 && steps[s].dep >= 0 && (uint32_t)steps[s].dep < s && steps[s].w)
            L.q_n[(uint32_t)steps[s].dep] = steps[s].w->K;
    for (uint32_t s = 0; s < n; s++) {
        if (!L.q_n[s]) continue;
        at = (at + 255) & ~(uint64_t)255;
        L.amax1_off[s] = (uint32_t)at; at += (uint64_t)16 * kAmaxStride * 4;
        L.amax2_off[s] = (uint32_t)at; at += (uint64_t)16 * kMaxPeers * 4;
        L.q_off[s] = (uint32_t)at; at += (uint64_t)packed_words(M) * L.q_n[s] * 4;
    }
    L.bytes = (at + 255) & ~(uint64_t)255;
    return L;
}

static int seq_create_impl(const sptmm_seq_step *steps, uint32_t n, uint32_t M, void *const *C_peers,
                           void *const *counter_peers, uint32_t n_peers, uint32_t my_rank, sptmm_seq **out)
{
    if (!steps || !out || n == 0) return fail(SPTMM_ERR_INVALID, "seq_create: null pointer or empty sequence");
    *out = nullptr;
    if (n_peers > kMaxPeers || (n_peers && (!C_peers || !counter_peers || my_rank >= n_peers)))
        return fail(SPTMM_ERR_INVALID, "seq_create: bad peer arguments (n_peers=%u, rank=%u)", n_peers, my_rank);
    if (M == 0 || M > 16) return fail(SPTMM_ERR_UNSUPPORTED, "seq_create: M=%u, the sequence kernel blocks 1..16 rows", M);
    int dev = 0, sms = 0, coop = 0;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    SPTMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    SPTMM_CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return fail(SPTMM_ERR_UNSUPPORTED, "seq_create: device cannot launch cooperatively");

    sptmm_seq *q = new (std::nothrow) sptmm_seq();
    if (!q) return fail(SPTMM_ERR_NOMEM, "seq_create: out of host memory");
    q->device = dev; q->nsteps = n; q->M = M; q->G = (uint32_t)sms;
    // rows per activation tile: 1, 4 or 16; sequences of the settled exchange also have an 8-row kernel
    bool any_settled = false;
    for (uint32_t s = 0; s < n; s++) any_settled = any_settled || steps[s].x_kind == 5;
    q->mt = M == 1 ? 1 : (M <= 4 ? 4 : ((M <= 8 && any_settled) ? 8 : 16));
    std::vector<SeqDesc> desc(n);
    std::vector<uint32_t> blk, col, tb, tc;
    uint32_t kmax = 0;
    for (uint32_t s = 0; s < n; s++) {
        const sptmm_seq_step &st = steps[s];
        const sptmm_weights *w = st.w;
        int rc = SPTMM_OK;
        if (!w || !st.X || (!st.C && !n_peers)) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u has a null pointer", s);
        else if (w->format != SPTMM_FMT_U16_V256) rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: step %u is not in the native u16 format", s);
        else if (w->device != dev || st.replica >= w->dev.size()) rc = fail(SPTMM_ERR_STATE, "seq_create: step %u weights are not uploaded to device %d (replica %u)", s, dev, st.replica);
        else if (st.x_kind > 5) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u x_kind %u", s, st.x_kind);
        else if (st.x_kind == 5 && (st.dep < 0 || st.X2)) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u (x_kind 5) needs a producer (dep) and takes no X2", s);
        else if (st.x_kind == 5 && ((w->K & 3) || (reinterpret_cast<uintptr_t>(st.X) & 15) || (st.ldx & 3) || (M == 1 && w->K > 14336) ||
                                    (w->K + (uint32_t)sms - 1) / (uint32_t)sms > 512))
            rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: step %u (x_kind 5) needs K a multiple of 4 (at most 14336 for one row), X 16-byte aligned and ldx a multiple of 4", s);
        else if (st.x_kind == 4 && (st.dep < 0 || st.X2)) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u (x_kind 4) needs a producer (dep) and takes no X2", s);
        else if (st.x_kind == 3 && (st.dep < 0 || st.X2)) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u (x_kind 3) needs a producer (dep) and takes no X2", s);
        else if (st.c_kind > 2 || (st.c_kind == 1 && (w->N & 1))) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u c_kind %u (pair sums need an even N)", s, st.c_kind);
        else if (st.x_kind != 0 && st.dep >= 0 && (uint32_t)st.dep < s && steps[(uint32_t)st.dep].c_kind == 2)
            rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u quantises the output of step %d, which holds de-quantised floats", s, st.dep);
        else if (st.c_kind == 2 && st.x_kind == 4) rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: step %u: a de-quantised output needs the step to know its input's scale (not x_kind 4)", s);
        else if (st.x_kind == 2 && st.dep < 0) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u reads tagged words but names no producer (dep)", s);
        else if (st.dep >= (int32_t)s) rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u depends on step %d, which does not precede it", s, st.dep);
        if (rc != SPTMM_OK) { seq_release(q); return rc; }
        SeqDesc &d = desc[s];
        d.idx = (const uint4 *)w->dev[st.replica][0];
        d.blk_off = (const uint32_t *)w->dev[st.replica][1];
        d.X = st.X; d.X2 = st.X2; d.C = (int32_t *)st.C; d.scale_out = st.scale_out;
        d.K = w->K; d.N = w->N;
        d.ldx = st.ldx ? st.ldx : w->K; d.ldx2 = st.ldx2 ? st.ldx2 : w->K; d.ldc = st.ldc ? st.ldc : w->N;
        d.uniform_nbl = w->uniform_nbl; d.x_kind = st.x_kind; d.dep = st.dep < 0 ? -1 : st.dep;
        d.c_kind = st.c_kind;
        d.ldc = st.ldc ? st.ldc : (st.c_kind == 1 ? w->N / 2 : w->N);
        for (uint32_t r = 0; r < kMaxPeers; r++) d.Cp[r] = r < n_peers ? (int32_t *)C_peers[(size_t)s * n_peers + r] : nullptr;
        if (n_peers) {
            for (uint32_t r = 0; r < n_peers; r++)
                if (!d.Cp[r]) { seq_release(q); return fail(SPTMM_ERR_INVALID, "seq_create: step %u has no output pointer for rank %u", s, r); }
            d.C = d.Cp[my_rank];
        }
        uint32_t mc = 1, mb = 0;
        plan_columns((const uint32_t *)w->arrays[1].data.data(), w->N, q->G, tb, tc, mc, mb, st.c_kind == 1 ? 2u : 1u);
        blk.insert(blk.end(), tb.begin(), tb.end());
        col.insert(col.end(), tc.begin(), tc.end());
        q->max_cols = std::max(q->max_cols, mc);
        kmax = std::max(kmax, w->K);
        q->stream_bytes += w->stream_bytes;
    }
    // Tagged exchange: a step with x_kind 2 makes the step it names in `dep` store tagged words.
    // Every step writing that buffer must then be tagged (a plain value could pass for a tag), and
    // nobody may wait for such a step through its counter, which it no longer bumps.
    {
        std::vector<char> tagged(n, 0);
        for (uint32_t s = 0; s < n; s++)
            if (steps[s].x_kind == 2 || steps[s].x_kind == 5) { tagged[(uint32_t)steps[s].dep] = 1; q->tagged = true; }
        int rc = SPTMM_OK;
        for (uint32_t s = 0; s < n && rc == SPTMM_OK; s++) {
            desc[s].release = tagged[s] ? 0 : 1;
            if (steps[s].x_kind == 3) { desc[(uint32_t)steps[s].dep].want_amax = 1; q->uses_amax = true; }
            if (tagged[s] && desc[s].c_kind == 2)
                rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u stores de-quantised floats, but a later step reads its output as tagged integers", s);
            if (tagged[s] && desc[s].c_kind == 1 && desc[s].K > 33000)
                rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: step %u: pair sums over K=%u rows do not fit a tagged word", s, desc[s].K);
            if (steps[s].x_kind != 2 && steps[s].x_kind != 5 && steps[s].x_kind != 4 && steps[s].dep >= 0 && tagged[(uint32_t)steps[s].dep])
                rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u waits for step %d, whose output is tagged for an x_kind 2 or 5 reader", s, steps[s].dep);
            if (!tagged[s]) continue;
            uint32_t m = 0, j = 0;
            for (uint32_t t = 0; t < n; t++)
                if (desc[t].C == desc[s].C) {
                    if (!tagged[t]) rc = fail(SPTMM_ERR_INVALID, "seq_create: steps %u and %u write the same buffer, but only one of them feeds an x_kind 2 reader", s, t);
                    if (t < s) j++;
                    m++;
                }
            desc[s].out_tag_m = m; desc[s].out_tag_j = j;
        }
        for (uint32_t s = 0; s < n && rc == SPTMM_OK; s++)
            if (steps[s].x_kind == 2 || steps[s].x_kind == 5) {
                const SeqDesc &pd = desc[(uint32_t)steps[s].dep];
                desc[s].in_tag_m = pd.out_tag_m; desc[s].in_tag_j = pd.out_tag_j;
                // the producer's rows are ldc wide and its columns (one shard of them, on several
                // GPUs) start somewhere inside the first row: accept any address within the rows
                const char *lo = (const char *)pd.C - (size_t)pd.ldc * 4, *hi = (const char *)pd.C + (size_t)M * pd.ldc * 4;
                const char *x = (const char *)steps[s].X, *x2 = (const char *)steps[s].X2;
                if (x < lo || x >= hi || (x2 && (x2 < lo || x2 >= hi)))
                    rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u reads tagged words outside the output of step %d", s, steps[s].dep);
            }
        if (rc != SPTMM_OK) { seq_release(q); return rc; }
    }

    // Producer-side quantiser: an x_kind 4 step makes the step it names in `dep` quantise the
    // columns it reads.  Its X names those columns inside the producer's output (that is how the
    // range is given); what the kernel reads instead is the producer's packed copy in the
    // synchronisation area, patched in below once that area's address is known.
    const SeqLayout layout = seq_layout(steps, n, M);
    {
        int rc = SPTMM_OK;
        bool any_q = false;
        for (uint32_t s = 0; s < n; s++) any_q = any_q || layout.q_n[s] != 0;
        if (any_q && (uint32_t)sms > kAmaxStride)
            rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: %d SMs, the row-maxima tables plan for at most %u", sms, kAmaxStride);
        for (uint32_t s = 0; s < n && rc == SPTMM_OK; s++) {
            if (steps[s].x_kind != 4) continue;
            const uint32_t pr = (uint32_t)steps[s].dep;
            SeqDesc &pd = desc[pr];
            const long long diff = (const char *)steps[s].X - (const char *)pd.C;
            if (diff % 4 || diff / 4 < -(1 << 24) || diff / 4 > (1 << 24))
                rc = fail(SPTMM_ERR_INVALID, "seq_create: step %u (x_kind 4) does not read inside the output of step %u", s, pr);
            else if (pd.q_n && (pd.q_n != desc[s].K || pd.q_0 != (int32_t)(diff / 4)))
                rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: steps reading step %u quantised must read the same columns", pr);
            else if (2ull * 127 * pd.K >= (1ull << 24))
                rc = fail(SPTMM_ERR_UNSUPPORTED, "seq_create: step %u: K=%u is too long for 24-bit row maxima", pr, pd.K);
            else {
                pd.q_n = desc[s].K; pd.q_0 = (int32_t)(diff / 4);
                pd.q_off = layout.q_off[pr]; pd.amax1_off = layout.amax1_off[pr]; pd.amax2_off = layout.amax2_off[pr];
                pd.q_scale_out = steps[s].scale_out;
                q->tagged = true;                       // the kernel variant that knows the exchanges
            }
        }
        // a step bumps its counter only if somebody waits for it there (the release stalls warp 0
        // until its stores have landed, on every rank)
        for (uint32_t s = 0; s < n; s++) {
            bool waited = false;
            for (uint32_t t = s + 1; t < n; t++)
                if (steps[t].dep == (int32_t)s && steps[t].x_kind != 2 && steps[t].x_kind != 4 && steps[t].x_kind != 5) waited = true;
            if (!waited) desc[s].release = 0;
        }
        if (rc != SPTMM_OK) { seq_release(q); return rc; }
    }

    // shared memory: X tile, column sums + scratch, then as many 1 KB ring slots per warp as fit
    const uint32_t nwarps = 16;               // consumer warps (one more warp produces)
    q->xs_bytes = (uint32_t)xs_bytes(kmax, (int)q->mt);
    // The settle phase runs in warps of its own, one step ahead, when that can overlap anything: tiles of
    // several rows, settled exchange, and a step list in which some step reads the output of a step
    // before the previous one (interleaved chains).  int8 inputs are then staged by the settle warps
    // too, which do not wait for step counters.
    {
        bool ahead = false, plain_ok = true;
        for (uint32_t s = 0; s < n; s++) {
            if (steps[s].x_kind == 5 && steps[s].dep + 2 <= (int32_t)s) ahead = true;
            if (steps[s].x_kind == 0 && steps[s].dep >= 0) plain_ok = false;
        }
        q->pipe = any_settled && q->mt >= 4 && ahead && plain_ok && 2 * (size_t)q->xs_bytes <= 120 * 1024;
    }
    const size_t tiles = q->pipe ? 2 * (size_t)q->xs_bytes : (size_t)q->xs_bytes;
    size_t fixed = tiles + (2 * (size_t)q->max_cols * q->mt + kRedInts) * 4;
    fixed = (fixed + 7) & ~(size_t)7;
    const size_t avail = 223 * 1024;      // minus static shared memory and the gap before the tile
    // 4 KB slots stream best; halve them while three of them per warp do not fit beside the X tile
    uint32_t slot_blocks = kMaxSlotBlocks;
    while (slot_blocks > 1 && fixed + 128 + (size_t)nwarps * 3 * (slot_blocks * 512 + 16) > avail) slot_blocks /= 2;
    const size_t slot_bytes = (size_t)slot_blocks * 512;
    q->slot_blocks = slot_blocks;
    if (fixed + 128 + (size_t)nwarps * 2 * (slot_bytes + 16) > avail) {
        const uint32_t mt = q->mt;
        seq_release(q);
        return fail(SPTMM_ERR_UNSUPPORTED, "seq_create: K=%u with %u-row blocking leaves no room for the weight rings", kmax, mt);
    }
    q->ring_slots = (uint32_t)std::min<size_t>(seq_ring_cap(), (avail - fixed - 128) / ((size_t)nwarps * (slot_bytes + 16)));
    size_t o = fixed + (size_t)nwarps * 2 * q->ring_slots * 8;
    o = (o + 127) & ~(size_t)127;
    q->smem = 1024 + o + (size_t)nwarps * q->ring_slots * slot_bytes;

    q->n_peers = n_peers; q->my_rank = my_rank;
    cudaError_t e = cudaSuccess;
    if (n_peers) {                    // counters live in peer-mapped memory the caller owns and zeroed
        for (uint32_t r = 0; r < n_peers; r++) {
            if (!counter_peers[r]) { seq_release(q); return fail(SPTMM_ERR_INVALID, "seq_create: no counters for rank %u", r); }
            q->counter_peers[r] = counter_peers[r];
        }
    } else {
        e = cudaMalloc(&q->d_counters, layout.bytes);
        if (e == cudaSuccess) e = cudaMemset(q->d_counters, 0, layout.bytes);
    }
    const char *own_area = (const char *)(n_peers ? counter_peers[my_rank] : q->d_counters);
    for (uint32_t s = 0; s < n; s++)
        if (steps[s].x_kind == 4) desc[s].X = own_area + desc[(uint32_t)steps[s].dep].q_off;
    if (e == cudaSuccess) e = cudaMalloc(&q->d_desc, n * sizeof(SeqDesc));
    if (e == cudaSuccess) e = cudaMemcpy(q->d_desc, desc.data(), n * sizeof(SeqDesc), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&q->d_blk, blk.size() * 4);
    if (e == cudaSuccess) e = cudaMemcpy(q->d_blk, blk.data(), blk.size() * 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&q->d_col, col.size() * 4);
    if (e == cudaSuccess) e = cudaMemcpy(q->d_col, col.data(), col.size() * 4, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMalloc(&q->d_status, 16);
    if (e == cudaSuccess) e = cudaMemset(q->d_status, 0, 16);
    {
        uint32_t k5 = 0;                                     // longest row any settled-exchange step reads
        for (uint32_t s = 0; s < n; s++)
            if (steps[s].x_kind == 5) k5 = std::max(k5, desc[s].K);
        if (k5 && q->mt > 1 && q->uses_amax) {
            seq_release(q);
            return fail(SPTMM_ERR_UNSUPPORTED, "seq_create: x_kind 3 and x_kind 5 steps of several rows cannot share a sequence (both keep row maxima per step)");
        }
        if (k5) {
            for (uint32_t s = 0; s < n; s++)
                if (steps[s].x_kind != 0 && steps[s].x_kind != 5) {
                    seq_release(q);
                    return fail(SPTMM_ERR_UNSUPPORTED, "seq_create: a sequence with x_kind 5 steps takes x_kind 0 and 5 only (step %u is %u)", s, steps[s].x_kind);
                }
            q->settled = true;
            if (q->mt > 1) q->uses_amax = true;              // the steps' row maxima live in that area
            q->xq_stride = (uint32_t)(((size_t)k5 * q->mt + 255) & ~(size_t)255);
            if (e == cudaSuccess) e = cudaMalloc(&q->d_xq, 2 * (size_t)q->xq_stride);
        }
    }
    if (e != cudaSuccess) { seq_release(q); return fail(SPTMM_ERR_CUDA, "seq_create: %s", cudaGetErrorString(e)); }
    *out = q;
    return SPTMM_OK;
}

// step counters (n x u64), then the row maxima (2 halves x n steps x 16 rows x u32)
// and two local arrival counters per step (x_kind 5)
static uint64_t seq_settle_offset(uint32_t n_steps) { return (uint64_t)n_steps * 8 + (uint64_t)2 * n_steps * 16 * 4; }
extern "C" uint64_t sptmm_seq_shared_bytes(uint32_t n_steps) { return seq_settle_offset(n_steps) + (uint64_t)n_steps * 16; }

extern "C" uint64_t sptmm_seq_shared_bytes_for(const sptmm_seq_step *steps, uint32_t n_steps, uint32_t M)
{
    if (!steps || n_steps == 0 || M == 0 || M > 16) return 0;
    return seq_layout(steps, n_steps, M).bytes;
}

extern "C" int sptmm_seq_create(const sptmm_seq_step *steps, uint32_t n, uint32_t M, sptmm_seq **out)
{
    return seq_create_impl(steps, n, M, nullptr, nullptr, 0, 0, out);
}

extern "C" int sptmm_seq_create_shared(const sptmm_seq_step *steps, uint32_t n, uint32_t M, void *const *C_peers,
                                       void *const *counter_peers, uint32_t n_peers, uint32_t my_rank, sptmm_seq **out)
{
    if (n_peers == 0) return fail(SPTMM_ERR_INVALID, "seq_create_shared: n_peers must be at least 1");
    return seq_create_impl(steps, n, M, C_peers, counter_peers, n_peers, my_rank, out);
}

template <int MT, int XV>
static int seq_launch_as(const sptmm_seq *q, const SeqParams &prm, cudaStream_t st);

template <int MT>
static int seq_launch(const sptmm_seq *q, const SeqParams &prm, cudaStream_t st)
{
    // every kernel variant carries only the exchanges its sequence uses (see k_seq); the plain one is
    // 0.7 us per step faster on the 6912x2560 sequence than one that knows them all
    if constexpr (MT >= 4) {
        if (q->settled && q->pipe) return seq_launch_as<MT, 3>(q, prm, st);
    }
    if (q->settled) return seq_launch_as<MT, 2>(q, prm, st);
    return (q->tagged || q->uses_amax) ? seq_launch_as<MT, 1>(q, prm, st) : seq_launch_as<MT, 0>(q, prm, st);
}

template <int MT, int XV>
static int seq_launch_as(const sptmm_seq *q, const SeqParams &prm, cudaStream_t st)
{
    static std::atomic<int> configured_device{-1};     // host threads may launch concurrently
    if (configured_device.load(std::memory_order_acquire) != q->device) {
        SPTMM_CUDA_TRY(cudaFuncSetAttribute(k_seq<MT, XV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        configured_device.store(q->device, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(q->G); cfg.blockDim = dim3(XV == 3 ? kPipeThreads : q->threads); cfg.dynamicSmemBytes = q->smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident at once, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    SPTMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, k_seq<MT, XV>, prm));
    return SPTMM_OK;
}

extern "C" int sptmm_seq_run(sptmm_seq *q, void *stream)
{
    if (!q) return fail(SPTMM_ERR_INVALID, "seq_run: null handle");
    int dev = -1;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != q->device) return fail(SPTMM_ERR_STATE, "seq_run: sequence lives on device %d, current device is %d", q->device, dev);
    q->epoch++;
    SeqParams prm;
    prm.desc = (const SeqDesc *)q->d_desc;
    prm.cta_blk = (const uint32_t *)q->d_blk;
    prm.cta_col = (const uint32_t *)q->d_col;
    prm.counters = (unsigned long long *)q->d_counters;
    prm.status = (uint32_t *)q->d_status;
#ifdef SPTMM_TUNING
    prm.trace = (unsigned long long *)q->d_trace;
#endif
    prm.n_peers = q->n_peers;
    for (uint32_t r = 0; r < kMaxPeers; r++) prm.counter_peers[r] = (unsigned long long *)q->counter_peers[r];
    if (q->n_peers) prm.counters = prm.counter_peers[q->my_rank];
    // a step is complete once every CTA of every rank has reported
    prm.target = (unsigned long long)q->G * q->epoch * (q->n_peers ? q->n_peers : 1);
    prm.nsteps = q->nsteps; prm.M = q->M; prm.max_cols = q->max_cols; prm.ring_slots = q->ring_slots;
    prm.xs_bytes = q->xs_bytes; prm.G = q->G; prm.slot_blocks = q->slot_blocks; prm.one = 1;
    prm.run_mod = (uint32_t)(q->epoch % 255);
    prm.run_parity = (uint32_t)(q->epoch & 1);
    prm.my_rank = q->my_rank;
    prm.settle = (unsigned long long *)((char *)prm.counters + seq_settle_offset(q->nsteps));
    prm.xq = (unsigned char *)q->d_xq; prm.xq_stride = q->xq_stride;
    prm.target_local = (unsigned long long)q->G * q->epoch;
    prm.poll_limit = q->poll_limit;
    // the row maxima sit behind the counters; a sequence without x_kind 3 steps never touches them
    for (uint32_t r = 0; r < kMaxPeers; r++)
        prm.amax_peers[r] = q->uses_amax && q->counter_peers[r] ? (uint32_t *)((char *)q->counter_peers[r] + (size_t)q->nsteps * 8) : nullptr;
    prm.amax = q->uses_amax ? (uint32_t *)((char *)prm.counters + (size_t)q->nsteps * 8) : nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    switch (q->mt) {
        case 1: return seq_launch<1>(q, prm, st);
        case 4: return seq_launch<4>(q, prm, st);
        case 8: return q->pipe ? seq_launch_as<8, 3>(q, prm, st) : seq_launch_as<8, 2>(q, prm, st);   // settled sequences only (see seq_create_impl)
        case 16: return seq_launch<16>(q, prm, st);
    }
    return fail(SPTMM_ERR_INVALID, "internal: row tile %u", q->mt);
}

extern "C" int sptmm_seq_status(sptmm_seq *q, uint32_t *status, uint64_t *stream_bytes)
{
    if (!q) return fail(SPTMM_ERR_INVALID, "seq_status: null handle");
    if (status) {
        SPTMM_CUDA_TRY(cudaDeviceSynchronize());
        SPTMM_CUDA_TRY(cudaMemcpy(status, q->d_status, 4, cudaMemcpyDeviceToHost));
    }
    if (stream_bytes) *stream_bytes = q->stream_bytes;
    return SPTMM_OK;
}

#ifdef SPTMM_TUNING
extern "C" int sptmm_seq_set_trace(sptmm_seq *q, void *dev_ptr)
{
    if (!q) return fail(SPTMM_ERR_INVALID, "seq_set_trace: null handle");
    q->d_trace = dev_ptr;
    return SPTMM_OK;
}
#endif

extern "C" int sptmm_seq_set_wait_limit(sptmm_seq *q, uint32_t polls)
{
    if (!q) return fail(SPTMM_ERR_INVALID, "seq_set_wait_limit: null handle");
    q->poll_limit = polls ? polls : 1u << 21;
    return SPTMM_OK;
}

extern "C" int sptmm_seq_free(sptmm_seq *q)
{
    seq_release(q);
    return SPTMM_OK;
}

// ---------------------------------------------------------------------------------------------
// A sequence run that allocates nothing.
//
// Some callers may not allocate device memory at the moment they need a matmul: code running
// inside a memory pool that was sized up front and closed, a real-time loop that forbids calls
// which can block on the allocator, or a host framework that owns every byte of the device and
// hands out only the buffers it was asked for.  For them the sequence kernel's scratch -- the
// step descriptors, the per-CTA plan, the step counters and the status word -- lives in the
// fixed array below instead of in memory obtained from cudaMalloc.  The array is part of the
// library image: every GPU that loads the library carries it until the process exits.
constexpr uint32_t kStaticMaxSteps = 16;      // steps per call
constexpr uint32_t kStaticMaxCtas = 256;      // SMs of the device
constexpr size_t kStaticDescOff = 0;
constexpr size_t kStaticBlkOff = (kStaticMaxSteps * sizeof(SeqDesc) + 255) & ~(size_t)255;
constexpr size_t kStaticColOff = kStaticBlkOff + (size_t)kStaticMaxSteps * (kStaticMaxCtas + 1) * 4;
constexpr size_t kStaticCtrOff = (kStaticColOff + (size_t)kStaticMaxSteps * (kStaticMaxCtas + 1) * 4 + 255) & ~(size_t)255;
constexpr size_t kStaticStatusOff = kStaticCtrOff + 256;
constexpr size_t kStaticBytes = kStaticStatusOff + 256;          // about 36 KB
static __device__ __align__(256) unsigned char g_seq_static_scratch[kStaticBytes];

extern "C" int sptmm_seq_run_static(const sptmm_seq_step *steps, uint32_t n, uint32_t M, void *stream,
                                    uint32_t *status_out)
{
    if (!steps || n == 0) return fail(SPTMM_ERR_INVALID, "seq_run_static: null pointer or empty sequence");
    if (n > kStaticMaxSteps)
        return fail(SPTMM_ERR_INVALID, "seq_run_static: %u steps, the fixed scratch holds at most %u", n, kStaticMaxSteps);
    if (M == 0 || M > 16) return fail(SPTMM_ERR_UNSUPPORTED, "seq_run_static: M=%u, the sequence kernel blocks 1..16 rows", M);
    int dev = 0, sms = 0;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(SPTMM_ERR_UNSUPPORTED, "seq_run_static: device ordinal %d", dev);

    // Once per device, with that device current: the array's name is only a stand-in on the host;
    // the address a kernel can use has to be asked for.
    static unsigned char *scratch_of[64] = {};
    static int sms_of[64] = {};
    static std::mutex setup_lock;                  // host threads may make their first calls at the same time
    unsigned char *scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(setup_lock);
        if (!scratch_of[dev]) {
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_seq_static_scratch);
            if (e != cudaSuccess || !p) return fail(SPTMM_ERR_CUDA, "seq_run_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            SPTMM_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            sms_of[dev] = sms;
            scratch_of[dev] = (unsigned char *)p;
        }
        sms = sms_of[dev];
        scratch = scratch_of[dev];
    }
    if ((uint32_t)sms > kStaticMaxCtas)
        return fail(SPTMM_ERR_UNSUPPORTED, "seq_run_static: %d SMs, the fixed scratch plans for at most %u", sms, kStaticMaxCtas);

    // host-side tables (host heap only), laid out exactly as the kernel reads them
    sptmm_seq q;                                   // a plain host object, nothing on the device
    q.device = dev; q.nsteps = n; q.M = M; q.G = (uint32_t)sms;
    q.mt = M == 1 ? 1 : (M <= 4 ? 4 : 16);
    std::vector<SeqDesc> desc(n);
    std::vector<uint32_t> blk, col, tb, tc;
    uint32_t kmax = 0;
    for (uint32_t s = 0; s < n; s++) {
        const sptmm_seq_step &st = steps[s];
        const sptmm_weights *w = st.w;
        if (!w || !st.X || !st.C) return fail(SPTMM_ERR_INVALID, "seq_run_static: step %u has a null pointer", s);
        if (w->format != SPTMM_FMT_U16_V256) return fail(SPTMM_ERR_UNSUPPORTED, "seq_run_static: step %u is not in the native u16 format", s);
        if (w->device != dev || st.replica >= w->dev.size()) return fail(SPTMM_ERR_STATE, "seq_run_static: step %u weights are not uploaded to device %d", s, dev);
        if (st.x_kind > 1 || st.c_kind != 0 || st.dep >= (int32_t)s) return fail(SPTMM_ERR_INVALID, "seq_run_static: step %u has a bad x_kind, c_kind or dep", s);
        SeqDesc &d = desc[s];
        d.idx = (const uint4 *)w->dev[st.replica][0];
        d.blk_off = (const uint32_t *)w->dev[st.replica][1];
        d.X = st.X; d.X2 = st.X2; d.C = (int32_t *)st.C; d.scale_out = st.scale_out;
        d.K = w->K; d.N = w->N;
        d.ldx = st.ldx ? st.ldx : w->K; d.ldx2 = st.ldx2 ? st.ldx2 : w->K; d.ldc = st.ldc ? st.ldc : w->N;
        d.uniform_nbl = w->uniform_nbl; d.x_kind = st.x_kind; d.dep = st.dep < 0 ? -1 : st.dep;
        for (uint32_t r = 0; r < kMaxPeers; r++) d.Cp[r] = nullptr;
        d.release = 1;
        uint32_t mc = 1, mb = 0;
        plan_columns((const uint32_t *)w->arrays[1].data.data(), w->N, q.G, tb, tc, mc, mb);
        blk.insert(blk.end(), tb.begin(), tb.end());
        col.insert(col.end(), tc.begin(), tc.end());
        q.max_cols = std::max(q.max_cols, mc);
        kmax = std::max(kmax, w->K);
    }
    const uint32_t nwarps = 16;
    q.xs_bytes = (uint32_t)xs_bytes(kmax, (int)q.mt);
    size_t fixed = q.xs_bytes + (2 * (size_t)q.max_cols * q.mt + kRedInts) * 4;
    fixed = (fixed + 7) & ~(size_t)7;
    const size_t avail = 223 * 1024;
    uint32_t slot_blocks = kMaxSlotBlocks;
    while (slot_blocks > 1 && fixed + 128 + (size_t)nwarps * 3 * (slot_blocks * 512 + 16) > avail) slot_blocks /= 2;
    const size_t slot_bytes = (size_t)slot_blocks * 512;
    q.slot_blocks = slot_blocks;
    if (fixed + 128 + (size_t)nwarps * 2 * (slot_bytes + 16) > avail)
        return fail(SPTMM_ERR_UNSUPPORTED, "seq_run_static: K=%u with %u-row blocking leaves no room for the weight rings", kmax, q.mt);
    q.ring_slots = (uint32_t)std::min<size_t>(seq_ring_cap(), (avail - fixed - 128) / ((size_t)nwarps * (slot_bytes + 16)));
    size_t o = fixed + (size_t)nwarps * 2 * q.ring_slots * 8;
    o = (o + 127) & ~(size_t)127;
    q.smem = 1024 + o + (size_t)nwarps * q.ring_slots * slot_bytes;

    // tables in, and what must start at zero cleared: the array keeps the previous call's contents
    cudaStream_t st = (cudaStream_t)stream;
    // The table copies below read host vectors that die with this call, and a status request waits
    // for the stream: neither survives being recorded into a graph, so a capturing stream is refused.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    SPTMM_CUDA_TRY(cudaStreamIsCapturing(st, &capturing));
    if (capturing != cudaStreamCaptureStatusNone)
        return fail(SPTMM_ERR_STATE, "seq_run_static: the stream is being captured; this call copies per-call tables from host memory and cannot be recorded");
    SPTMM_CUDA_TRY(cudaMemcpyAsync(scratch + kStaticDescOff, desc.data(), n * sizeof(SeqDesc), cudaMemcpyHostToDevice, st));
    SPTMM_CUDA_TRY(cudaMemcpyAsync(scratch + kStaticBlkOff, blk.data(), blk.size() * 4, cudaMemcpyHostToDevice, st));
    SPTMM_CUDA_TRY(cudaMemcpyAsync(scratch + kStaticColOff, col.data(), col.size() * 4, cudaMemcpyHostToDevice, st));
    SPTMM_CUDA_TRY(cudaMemsetAsync(scratch + kStaticCtrOff, 0, kStaticBytes - kStaticCtrOff, st));

    SeqParams prm;
    prm.desc = (const SeqDesc *)(scratch + kStaticDescOff);
    prm.cta_blk = (const uint32_t *)(scratch + kStaticBlkOff);
    prm.cta_col = (const uint32_t *)(scratch + kStaticColOff);
    prm.counters = (unsigned long long *)(scratch + kStaticCtrOff);
    for (uint32_t r = 0; r < kMaxPeers; r++) prm.counter_peers[r] = nullptr;
    prm.n_peers = 0;
    prm.status = (uint32_t *)(scratch + kStaticStatusOff);
#ifdef SPTMM_TUNING
    prm.trace = nullptr;
#endif
    prm.target = q.G;                              // counters were just cleared: one run's worth
    prm.nsteps = n; prm.M = M; prm.max_cols = q.max_cols; prm.ring_slots = q.ring_slots;
    prm.xs_bytes = q.xs_bytes; prm.G = q.G; prm.slot_blocks = q.slot_blocks; prm.one = 1; prm.run_mod = 0; prm.run_parity = 0; prm.amax = nullptr; prm.my_rank = 0;
    prm.settle = nullptr; prm.xq = nullptr; prm.xq_stride = 0; prm.target_local = 0; prm.poll_limit = 1u << 21;
    for (uint32_t r = 0; r < kMaxPeers; r++) prm.amax_peers[r] = nullptr;
    int rc = SPTMM_OK;
    switch (q.mt) {
        case 1: rc = seq_launch<1>(&q, prm, st); break;
        case 4: rc = seq_launch<4>(&q, prm, st); break;
        default: rc = seq_launch<16>(&q, prm, st); break;
    }
    q.device = -1;                                 // the host object owns nothing to release
    if (rc != SPTMM_OK) return rc;
    if (status_out) {
        SPTMM_CUDA_TRY(cudaStreamSynchronize(st));
        SPTMM_CUDA_TRY(cudaMemcpy(status_out, scratch + kStaticStatusOff, 4, cudaMemcpyDeviceToHost));
        if (*status_out) return fail(SPTMM_ERR_STATE, "seq_run_static: a bounded wait ran out (status %u)", *status_out);
    }
    return SPTMM_OK;
}
