// kernels_native.cu -- the B200 kernel for the native u16 format (SPTMM_FMT_U16_V256).
//
// Work it replaces: rowWiseSplit3Small4 (main.cu:556-594), one 32-thread CTA per column with
// two-byte index loads and byte gathers through L1, re-streaming every index once per row of X.
//
// Design.  The encoded matrix is one contiguous run of 512-byte blocks (256 sorted row indices
// of one column and one sign, see host_encode.cpp).  A plan made at upload time gives CTA i a
// contiguous range of whole columns with an equal share of blocks; the plan travels in the
// kernel parameters, so no global load precedes the first weight load.  Inside the CTA each
// warp takes an equal contiguous slice of those blocks.
//
// The kernel is a chain of latencies unless every byte is requested at once, so at entry each
// warp requests its whole slice: the first P blocks with 16-byte loads into registers, the rest
// with bulk copies (cp.async.bulk, completion on an mbarrier) into a warp-private, double-
// buffered staging area in shared memory.  Only then does it wait for the previous kernel in
// the stream (programmatic dependent launch); with two such CTAs resident per SM, DRAM streams
// this matrix while the previous kernel is still gathering.  A call launched without that
// overlap knows its activations are final at entry and asks for them BEFORE the weights (behind
// the weight requests they would arrive last, and no gather can start without them).
// The activation tile sits transposed in shared memory, so one gather serves MT rows of X and
// the index stream is read once for up to 16 rows.  Nothing is multiplied.
//
// A warp's slice can start and end inside a column.  Integer sums are order-free, so every
// finished list is added to its column's slot with a shared-memory atomic.  Floating-point sums
// for a warp's first and last column go to per-warp slots that are folded in warp order after a
// barrier (all other columns are owned by one warp), so results do not depend on scheduling.
// Every wait on an mbarrier is bounded; if one runs out the kernel raises a status word and
// returns instead of hanging.
#include <algorithm>
#include <atomic>

#include "device_common.cuh"

namespace sptmm {

constexpr int kMaxGrid = (int)kMaxPlanCtas;
constexpr int kMaxWarps = 16;
constexpr uint32_t kDeltaBlockBytes = 304;     // 256 offsets, 8 bases, 8 counts, padding (SPTMM_FMT_DELTA_LANE)

struct NativeParams {
    const uint4 *idx;            // total_blocks * 32 vectors
    const uint32_t *blk_off;     // 2N+1
    const void *X;
    void *C;
#ifdef SPTMM_TUNING
    unsigned long long *trace;   // optional: 8 timestamps per CTA for the first trace_ctas CTAs
    uint32_t trace_ctas;
#endif
    uint32_t *status;            // device word: set non-zero if a bounded wait ran out
    uint32_t K, N, M;
    uint32_t max_cols;
    uint32_t x_colmajor, c_colmajor;
    uint32_t uniform_nbl;        // blocks per list when every list has the same count, else 0
    uint32_t one;                // always 1: a multiplier the compiler cannot fold (LaneAcc::add)
    uint32_t x_early;            // X is final when the kernel starts (no programmatic overlap with its producer)
    // split-K over GPUs: n_peers > 0 makes the epilogue add each column's partial sum to the buffer
    // of the rank that owns the column (columns col_bound[r] .. col_bound[r+1] belong to rank r)
    uint32_t n_peers;
    uint32_t col_bound[9];
    void *Cp[8];
    // de-quantising epilogue (int8 activations only): store float(sum) * (row_scale[m] * out_scale)
    uint32_t scaled;
    const float *row_scale;      // per row of X, or null for 1
    float out_scale;
    uint32_t ldx;                // elements between rows of a row-major X (a K-tile of a wider matrix: the full width)
    uint32_t accumulate;         // 1: add to C instead of storing (the second and later K-tiles of a matrix)
    uint32_t half_blocks;        // blocks per half of a warp's staging area
    uint32_t stage_blocks;       // blocks of staging area per warp (one or two halves)
    uint32_t stage_off;          // byte offset of the staging area in dynamic shared memory
    uint32_t cta_blk[kMaxGrid + 1];   // block boundaries: CTA i owns blocks [cta_blk[i], cta_blk[i+1])
    uint32_t cta_col[kMaxGrid + 1];   // column boundaries: CTA i owns columns [cta_col[i], cta_col[i+1])
};

// Timestamps for kernel timelines exist only in the tuning build.
#ifdef SPTMM_TUNING
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define SPTMM_STAMP(slot) do { if (tracing) p.trace[blockIdx.x * 8 + (slot)] = global_ns(); } while (0)
#else
#define SPTMM_STAMP(slot) do { } while (0)
#endif

__device__ __forceinline__ uint4 ld_weights16(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// bulk copy global -> this CTA's shared memory, completion counted on `bar` (one elected lane)
__device__ __forceinline__ void bulk_fetch(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// returns false if the barrier did not complete the phase within the iteration limit
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < (1u << 22) && !done; spin++)
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}

template <int DT, int MT, int P, int MINB>
__global__ void __launch_bounds__(512, MINB) k_u16_v256(const __grid_constant__ NativeParams p)
{
    using acc_t = typename ActTraits<DT>::acc;
    constexpr int RB = MT * ActTraits<DT>::size;
    constexpr bool kInt = DT == SPTMM_I8;
    constexpr bool kDelta = P == 0;              // SPTMM_FMT_DELTA_LANE: 304-byte blocks, all through shared memory
    constexpr uint32_t BB = kDelta ? kDeltaBlockBytes : 512u;
    extern __shared__ __align__(16) unsigned char dyn_smem[];

    pdl_launch_dependents();     // the next kernel may start its own weight requests right away
    unsigned char *smem = tile_base(dyn_smem);     // everything below is laid out from the tile's fixed address
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const uint32_t b0 = p.cta_blk[blockIdx.x], b1 = p.cta_blk[blockIdx.x + 1];
    const uint32_t c0 = p.cta_col[blockIdx.x], c1 = p.cta_col[blockIdx.x + 1];
    const uint32_t ncols = c1 - c0, nlists = 2 * ncols;
    const uint32_t nb = b1 - b0;
    const uint32_t wb0 = b0 + (uint32_t)(((uint64_t)nb * warp) / nwarps);
    const uint32_t wb1 = b0 + (uint32_t)(((uint64_t)nb * (warp + 1)) / nwarps);
    const uint32_t n = wb1 - wb0;
    const uint32_t nbl = p.uniform_nbl;
#ifdef SPTMM_TUNING
    const bool tracing = p.trace != nullptr && blockIdx.x < p.trace_ctas && blockIdx.y == 0 && tid == 33;   // a lane that issues no fences or copies
#endif
    SPTMM_STAMP(0);

    // ---- list boundaries (only needed when lists differ in length): ask for them first, so the
    // answer is not queued behind the weight stream
    uint32_t off_r0 = 0, off_r1 = 0;
    if (nbl == 0) {
        if (tid <= nlists) off_r0 = __ldg(p.blk_off + 2 * (size_t)c0 + tid);
        if (tid + blockDim.x <= nlists) off_r1 = __ldg(p.blk_off + 2 * (size_t)c0 + tid + blockDim.x);
    }

    // ---- weights do not depend on the previous kernel: request the whole slice now
    const uint32_t H = p.half_blocks;
    const uint32_t nreg = min(n, (uint32_t)P);
    const uint32_t nstaged = n - nreg;
    const uint32_t nrounds = H ? (nstaged + H - 1) / H : 0;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + p.stage_off) + 2 * warp;
    const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(bars);
    const uint4 *wstage = reinterpret_cast<const uint4 *>(smem + p.stage_off + 256 + (size_t)warp * p.stage_blocks * BB);
    const uint32_t wstage_a = (uint32_t)__cvta_generic_to_shared(wstage);
    const unsigned char *slice_b = reinterpret_cast<const unsigned char *>(p.idx) + (size_t)wb0 * BB;
    const uint4 *slice = reinterpret_cast<const uint4 *>(slice_b);
    auto issue_round = [&](uint32_t r) {          // lane 0 only
        const uint32_t cnt = min(H, nstaged - r * H);
        bulk_fetch(wstage_a + (r & 1) * H * BB, slice_b + (size_t)(nreg + r * H) * BB, cnt * BB, bar_a + 8 * (r & 1));
    };
    uint4 buf[P ? P : 1];
    auto request_weights = [&]() {
        if (lane == 0 && nrounds) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a + 8) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_round(0);
            if (nrounds > 1) issue_round(1);
        }
#pragma unroll
        for (int i = 0; i < P; i++)
            if ((uint32_t)i < nreg) buf[i] = ld_weights16(slice + (size_t)i * 32 + lane);
    };

    // ---- A call that does not overlap its producer asks for X FIRST: behind the ~140 KB of weight
    // requests an SM has in flight the activations would arrive last, and no gather can start
    // without them.  One row (MT == 1) waits in registers while the weights are requested; wider
    // tiles are transposed into shared memory before the weights are requested.
    const uint32_t m0 = blockIdx.y * MT;
    const uint32_t mv = min((uint32_t)MT, p.M - m0);
    constexpr uint32_t ES = ActTraits<DT>::size;
    const unsigned char *xrow = reinterpret_cast<const unsigned char *>(p.X) + (size_t)m0 * p.ldx * ES;
    const uint32_t xvec = (p.K * ES) / 16;
    const bool x_regs = MT == 1 && p.x_early && !p.x_colmajor && (p.K * ES) % 16 == 0 &&
                        (reinterpret_cast<uintptr_t>(xrow) & 15) == 0 && xvec <= 2 * blockDim.x;
    const bool x_first = p.x_early && !x_regs;
    [[maybe_unused]] uint4 xr0 = make_uint4(0, 0, 0, 0), xr1 = make_uint4(0, 0, 0, 0);
    if constexpr (MT == 1) {
        if (x_regs) {
            if (tid < xvec) xr0 = __ldg(reinterpret_cast<const uint4 *>(xrow) + tid);
            if (tid + blockDim.x < xvec) xr1 = __ldg(reinterpret_cast<const uint4 *>(xrow) + tid + blockDim.x);
        }
    }
    if (!x_first) request_weights();

    // ---- shared memory carve-up
    unsigned char *xs = smem;
    uint32_t *off_s = reinterpret_cast<uint32_t *>(smem + xs_bytes(p.K, RB));      // nlists+1
    acc_t *c_s = reinterpret_cast<acc_t *>(off_s + 2 * p.max_cols + 1 + ((2 * p.max_cols + 1) & 1));
    acc_t *head_s = c_s + (size_t)p.max_cols * MT;                                  // nwarps*MT
    acc_t *tail_s = head_s + (size_t)nwarps * MT;                                   // nwarps*MT
    uint32_t *hcol_s = reinterpret_cast<uint32_t *>(tail_s + (size_t)nwarps * MT);  // nwarps
    uint32_t *tcol_s = hcol_s + nwarps;

    if (nbl == 0) {
        if (tid <= nlists) off_s[tid] = off_r0;
        if (tid + blockDim.x <= nlists) off_s[tid + blockDim.x] = off_r1;
        for (uint32_t i = tid + 2 * blockDim.x; i <= nlists; i += blockDim.x) off_s[i] = p.blk_off[2 * (size_t)c0 + i];
    }
    for (uint32_t i = tid; i < ncols * MT; i += blockDim.x) c_s[i] = acc_t(0);
    if (!kInt)
        for (uint32_t i = tid; i < nwarps * MT; i += blockDim.x) { head_s[i] = acc_t(0); tail_s[i] = acc_t(0); }

    pdl_wait_prior_grid();
    SPTMM_STAMP(1);

    if (x_regs) {
        if constexpr (MT == 1) {
            if (tid < xvec) reinterpret_cast<uint4 *>(xs)[tid] = xr0;
            if (tid + blockDim.x < xvec) reinterpret_cast<uint4 *>(xs)[tid + blockDim.x] = xr1;
            if (tid < ES) xs[(size_t)p.K * ES + tid] = 0;                     // the zero row
        }
    } else {
        stage_x<DT, MT, LaneAcc<DT, MT>::kBiased>(xs, p.X, p.K, p.M, m0, mv, p.x_colmajor != 0, p.ldx);
    }
    if (x_first) request_weights();
    __syncthreads();
    SPTMM_STAMP(2);

    if (n) {
        // local index (relative to list 2*c0) of the list that holds block wb0, and of wb1-1
        uint32_t li, llast, bound;
        if (nbl) {
            li = wb0 / nbl - 2 * c0;
            llast = (wb1 - 1) / nbl - 2 * c0;
            bound = (wb0 / nbl + 1) * nbl;
        } else {
            li = 0; llast = 0;
            for (uint32_t r = 1; r <= nlists; r += 32) {          // warp-uniform trip count
                const uint32_t i = r + lane;
                const uint32_t o = i <= nlists ? off_s[i] : 0xffffffffu;
                li += __popc(__ballot_sync(0xffffffffu, o <= wb0));
                llast += __popc(__ballot_sync(0xffffffffu, o <= wb1 - 1));
            }
            bound = off_s[li + 1];
        }
        const uint32_t first_col = li >> 1, last_col = llast >> 1;
        if (!kInt && lane == 0) { hcol_s[warp] = first_col; tcol_s[warp] = last_col; }

        LaneAcc<DT, MT> acc;
        acc.clear(p.one);
        bool dirty = false;

        [[maybe_unused]] PendingSums<MT> done;          // integer sums only (see device_common.cuh)
        done.clear();
        auto flush = [&]() {
            const uint32_t col = li >> 1;
            acc.finish();
            if constexpr (kInt) {
                done.push(acc.v, col, (li & 1) != 0, reinterpret_cast<int *>(c_s), lane);
            } else {
                // floats: the same butterfly (a fixed order of additions, so results repeat from run to
                // run); lane l ends with row l / (32/MT), and one lane per row adds it where it belongs
                constexpr uint32_t G = 32 / MT;
                acc_t sum = TransposeSum<acc_t, MT>::run(acc.v, lane, 16);
                sum = (li & 1) ? -sum : sum;
                acc_t *dst = col == first_col ? head_s + warp * MT : (col == last_col ? tail_s + warp * MT : c_s + col * MT);
                if ((lane & (G - 1)) == 0) dst[lane / G] += sum;
#pragma unroll
                for (int m = 0; m < MT; m++) acc.v[m] = acc_t(0);
            }
        };
        auto consume = [&](const uint4 v, const uint32_t b) {
            if (b >= bound) {                       // crossed into another list (rare)
                do {
                    if (dirty) { flush(); dirty = false; }
                    li++;
                    bound = nbl ? bound + nbl : off_s[li + 1];
                } while (b >= bound);
            }
            dirty = true;
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

        // two blocks at once when both lie inside the current list: sixteen independent gathers
        auto consume2 = [&](const uint4 v0, const uint4 v1, const uint32_t b) {
            if (b + 1 < bound) {
                dirty = true;
                acc.reserve(16);
                acc.add(v0.x & 0xffffu);
                acc.add(v1.x & 0xffffu);
                acc.add(v0.x >> 16);
                acc.add(v1.x >> 16);
                acc.add(v0.y & 0xffffu);
                acc.add(v1.y & 0xffffu);
                acc.add(v0.y >> 16);
                acc.add(v1.y >> 16);
                acc.add(v0.z & 0xffffu);
                acc.add(v1.z & 0xffffu);
                acc.add(v0.z >> 16);
                acc.add(v1.z >> 16);
                acc.add(v0.w & 0xffffu);
                acc.add(v1.w & 0xffffu);
                acc.add(v0.w >> 16);
                acc.add(v1.w >> 16);
            } else {
                consume(v0, b);
                consume(v1, b + 1);
            }
        };

        // A lane-delta block (SPTMM_FMT_DELTA_LANE, see host_encode.cpp): eight gather steps; step
        // t gathers rows base[t] + off[lane][t] for the first cnt[t] lanes.  Blocks whose steps
        // are all full (every block but a list's last, and steps cut short by a gap of more than
        // 255 rows) take the branch without per-lane tests; idle lanes read the zero row.
        auto consume_delta = [&](const uint32_t blk, const uint32_t b) {       // blk: shared-space address
            if (b >= bound) {
                do {
                    if (dirty) { flush(); dirty = false; }
                    li++;
                    bound = nbl ? bound + nbl : off_s[li + 1];
                } while (b >= bound);
            }
            dirty = true;
            acc.reserve(8);
            const uint2 off = lds64(blk + 8 * lane);
            const uint4 ba = lds128(blk + 256), bb = lds128(blk + 272);
            const uint2 cn = lds64(blk + 288);
            if (cn.x == 0x20202020u && cn.y == 0x20202020u) {
                acc.add(ba.x + __byte_perm(off.x, 0u, 0x4440));
                acc.add(ba.y + __byte_perm(off.x, 0u, 0x4441));
                acc.add(ba.z + __byte_perm(off.x, 0u, 0x4442));
                acc.add(ba.w + __byte_perm(off.x, 0u, 0x4443));
                acc.add(bb.x + __byte_perm(off.y, 0u, 0x4440));
                acc.add(bb.y + __byte_perm(off.y, 0u, 0x4441));
                acc.add(bb.z + __byte_perm(off.y, 0u, 0x4442));
                acc.add(bb.w + __byte_perm(off.y, 0u, 0x4443));
            } else {
                const uint32_t base[8] = {ba.x, ba.y, ba.z, ba.w, bb.x, bb.y, bb.z, bb.w};
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    const uint32_t o = ((t < 4 ? off.x : off.y) >> (8 * (t & 3))) & 0xffu;
                    const uint32_t c = ((t < 4 ? cn.x : cn.y) >> (8 * (t & 3))) & 0xffu;
                    acc.add(lane < c ? base[t] + o : p.K);
                }
            }
        };

        // two full blocks of one list at once: sixteen independent gathers in flight
        auto consume_delta2 = [&](const uint32_t blk0, const uint32_t blk1, const uint32_t b) {
            if (b + 1 < bound) {
                const uint2 o0 = lds64(blk0 + 8 * lane), o1 = lds64(blk1 + 8 * lane);
                const uint4 a0 = lds128(blk0 + 256), b0v = lds128(blk0 + 272), a1 = lds128(blk1 + 256), b1v = lds128(blk1 + 272);
                const uint2 c0v = lds64(blk0 + 288), c1v = lds64(blk1 + 288);
                if (c0v.x == 0x20202020u && c0v.y == 0x20202020u && c1v.x == 0x20202020u && c1v.y == 0x20202020u) {
                    dirty = true;
                    acc.reserve(16);
                    acc.add(a0.x + __byte_perm(o0.x, 0u, 0x4440));
                    acc.add(a1.x + __byte_perm(o1.x, 0u, 0x4440));
                    acc.add(a0.y + __byte_perm(o0.x, 0u, 0x4441));
                    acc.add(a1.y + __byte_perm(o1.x, 0u, 0x4441));
                    acc.add(a0.z + __byte_perm(o0.x, 0u, 0x4442));
                    acc.add(a1.z + __byte_perm(o1.x, 0u, 0x4442));
                    acc.add(a0.w + __byte_perm(o0.x, 0u, 0x4443));
                    acc.add(a1.w + __byte_perm(o1.x, 0u, 0x4443));
                    acc.add(b0v.x + __byte_perm(o0.y, 0u, 0x4440));
                    acc.add(b1v.x + __byte_perm(o1.y, 0u, 0x4440));
                    acc.add(b0v.y + __byte_perm(o0.y, 0u, 0x4441));
                    acc.add(b1v.y + __byte_perm(o1.y, 0u, 0x4441));
                    acc.add(b0v.z + __byte_perm(o0.y, 0u, 0x4442));
                    acc.add(b1v.z + __byte_perm(o1.y, 0u, 0x4442));
                    acc.add(b0v.w + __byte_perm(o0.y, 0u, 0x4443));
                    acc.add(b1v.w + __byte_perm(o1.y, 0u, 0x4443));
                    return;
                }
            }
            consume_delta(blk0, b);
            consume_delta(blk1, b + 1);
        };

        // the blocks that came straight into registers
        if constexpr (!kDelta) {
#pragma unroll
            for (int i = 0; i + 1 < P; i += 2) {
                if ((uint32_t)i + 1 < nreg) consume2(buf[i], buf[i + 1], wb0 + i);
                else if ((uint32_t)i < nreg) consume(buf[i], wb0 + i);
            }
        }

        // the staged blocks, round by round; a finished half is refilled two rounds ahead
        bool ok = true;
        for (uint32_t r = 0; r < nrounds; r++) {
            ok = bounded_wait(bar_a + 8 * (r & 1), (r >> 1) & 1);
            if (!ok) break;
            const uint32_t cnt = min(H, nstaged - r * H);
            const uint32_t bfirst = wb0 + nreg + r * H;
            if constexpr (kDelta) {
                const uint32_t half_a = wstage_a + (r & 1) * H * BB;
                uint32_t j = 0;
                for (; j + 1 < cnt; j += 2) consume_delta2(half_a + j * BB, half_a + (j + 1) * BB, bfirst + j);
                if (j < cnt) consume_delta(half_a + j * BB, bfirst + j);
            } else {
                const uint4 *half = wstage + (size_t)(r & 1) * H * 32 + lane;
                uint32_t j = 0;
                for (; j + 1 < cnt; j += 2) consume2(half[(size_t)j * 32], half[(size_t)(j + 1) * 32], bfirst + j);
                if (j < cnt) consume(half[(size_t)j * 32], bfirst + j);
            }
            if (r + 2 < nrounds) {
                __syncwarp();
                if (lane == 0) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue_round(r + 2);
                }
            }
        }
        // report, do not hang (a plain store: every writer stores the same 1, and the word may live
        // in mapped host memory, where atomics are not available on every platform)
        if (!ok && lane == 0 && p.status) *reinterpret_cast<volatile uint32_t *>(p.status) = 1u;
        if (dirty) flush();
        if constexpr (kInt) done.drain(reinterpret_cast<int *>(c_s), lane);
    } else if (!kInt && lane == 0) {
        hcol_s[warp] = 0xffffffffu; tcol_s[warp] = 0xffffffffu;
    }
    __syncthreads();
    SPTMM_STAMP(3);

    // ---- write the CTA's columns; floats first fold the per-warp edge sums in warp order
    acc_t *C = reinterpret_cast<acc_t *>(p.C);
    for (uint32_t i = tid; i < ncols * mv; i += blockDim.x) {
        const uint32_t m = i / ncols, col = i - m * ncols;
        acc_t v = c_s[col * MT + m];
        if constexpr (!kInt) {
#pragma unroll
            for (uint32_t w = 0; w < (uint32_t)kMaxWarps; w++) {
                if (w < nwarps) {
                    const uint32_t hc = hcol_s[w], tc = tcol_s[w];
                    const acc_t hv = head_s[w * MT + m], tv = tail_s[w * MT + m];
                    v += hc == col ? hv : (tc == col ? tv : acc_t(0));
                }
            }
        }
        if (p.n_peers) {
            // fused reduce-scatter: the sum goes to the column's owner (a plain reduction; over
            // NVLink when the owner is a peer)
            const uint32_t gcol = c0 + col;
            uint32_t r = 0;
            while (r + 1 < p.n_peers && gcol >= p.col_bound[r + 1]) r++;
            const uint32_t width = p.col_bound[r + 1] - p.col_bound[r];
            atomicAdd(reinterpret_cast<acc_t *>(p.Cp[r]) + (size_t)(m0 + m) * width + (gcol - p.col_bound[r]), v);
            continue;
        }
        const size_t o = p.c_colmajor ? (size_t)(c0 + col) * p.M + m0 + m : (size_t)(m0 + m) * p.N + c0 + col;
        if constexpr (kInt) {
            if (p.scaled) {          // the sum is exact in fp32 (|sum| <= 127 K < 2^23); one product of the two scales, one of the sum
                const float sc = (p.row_scale ? __ldg(p.row_scale + m0 + m) : 1.0f) * p.out_scale;
                reinterpret_cast<float *>(p.C)[o] = (float)v * sc;
                continue;
            }
        }
        if (p.accumulate) C[o] += v;        // K-tiles of one matrix run one after the other on the stream
        else C[o] = v;
    }
    SPTMM_STAMP(4);
}

// ---------------------------------------------------------------------------------------------

static size_t native_smem(uint32_t K, int rb, int mt, uint32_t max_cols, uint32_t nwarps)
{
    size_t s = xs_bytes(K, rb);
    size_t off_words = 2 * (size_t)max_cols + 1;
    off_words += off_words & 1;
    s += off_words * 4;
    s += (size_t)max_cols * mt * 4;
    s += 2 * (size_t)nwarps * mt * 4;
    s += 2 * (size_t)nwarps * 4;
    return (s + 127) & ~(size_t)127;       // the staging area (barriers, then blocks) starts here
}

template <int DT, int MT, int P, int MINB>
static int launch_one(const NativeParams &prm, dim3 grid, uint32_t threads, size_t smem, bool pdl, cudaStream_t st)
{
    static std::atomic<int> configured_device{-1};     // host threads may launch concurrently
    int dev = 0;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (configured_device.load(std::memory_order_acquire) != dev) {
        SPTMM_CUDA_TRY(cudaFuncSetAttribute(k_u16_v256<DT, MT, P, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        SPTMM_CUDA_TRY(cudaFuncSetAttribute(k_u16_v256<DT, MT, P, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                            cudaSharedmemCarveoutMaxShared));
        configured_device.store(dev, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    SPTMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, k_u16_v256<DT, MT, P, MINB>, prm));
    return SPTMM_OK;
}

// blocks a warp takes straight into registers (the rest of its slice goes through shared memory)
static int prefetch_depth(int mt, bool wide)
{
    const int t = wide ? 8 : tune().prefetch;
    if (mt == 1) return t >= 16 ? 16 : (t <= 4 ? 4 : 8);
    if (mt == 4) return t <= 4 ? 4 : 8;
    return mt == 2 ? 8 : 4;
}

template <int DT>
static int launch_dtype(const NativeParams &prm, int mt, int pd, bool wide, dim3 grid, uint32_t threads, size_t smem, bool pdl, cudaStream_t st)
{
    if (pd == 0)                      // lane-delta blocks: everything goes through shared memory
        switch (mt) {
            case 1: return wide ? launch_one<DT, 1, 0, 1>(prm, grid, threads, smem, pdl, st) : launch_one<DT, 1, 0, 2>(prm, grid, threads, smem, pdl, st);
            case 2: return wide ? launch_one<DT, 2, 0, 1>(prm, grid, threads, smem, pdl, st) : launch_one<DT, 2, 0, 2>(prm, grid, threads, smem, pdl, st);
            case 4: return wide ? launch_one<DT, 4, 0, 1>(prm, grid, threads, smem, pdl, st) : launch_one<DT, 4, 0, 2>(prm, grid, threads, smem, pdl, st);
            case 8: return launch_one<DT, 8, 0, 1>(prm, grid, threads, smem, pdl, st);
            case 16: return launch_one<DT, 16, 0, 1>(prm, grid, threads, smem, pdl, st);
        }
    if (wide)                         // one CTA per SM: no reason to cap registers at two CTAs' worth
        switch (mt) {
            case 1: return launch_one<DT, 1, 8, 1>(prm, grid, threads, smem, pdl, st);
            case 2: return launch_one<DT, 2, 8, 1>(prm, grid, threads, smem, pdl, st);
            case 4: return launch_one<DT, 4, 8, 1>(prm, grid, threads, smem, pdl, st);
            case 8: return launch_one<DT, 8, 4, 1>(prm, grid, threads, smem, pdl, st);
            case 16: return launch_one<DT, 16, 4, 1>(prm, grid, threads, smem, pdl, st);
        }
    switch (mt) {
        case 1:
            if (pd == 16) return launch_one<DT, 1, 16, 1>(prm, grid, threads, smem, pdl, st);
            if (pd == 4) return launch_one<DT, 1, 4, 2>(prm, grid, threads, smem, pdl, st);
            return launch_one<DT, 1, 8, 2>(prm, grid, threads, smem, pdl, st);
        case 2: return launch_one<DT, 2, 8, 2>(prm, grid, threads, smem, pdl, st);
        case 4:
            if (pd == 4) return launch_one<DT, 4, 4, 2>(prm, grid, threads, smem, pdl, st);
            return launch_one<DT, 4, 8, 2>(prm, grid, threads, smem, pdl, st);
        case 8: return launch_one<DT, 8, 4, 1>(prm, grid, threads, smem, pdl, st);
        case 16: return launch_one<DT, 16, 4, 1>(prm, grid, threads, smem, pdl, st);
    }
    return fail(SPTMM_ERR_INVALID, "internal: row tile %d", mt);
}

#ifdef SPTMM_TUNING
static unsigned long long *g_trace = nullptr;
void set_trace_buffer(unsigned long long *dev_ptr) { g_trace = dev_ptr; }
#endif

static int launch_native(const GemvArgs &a, const bool delta)
{
    const sptmm_weights &w = *a.w;
    const size_t bb = delta ? kDeltaBlockBytes : 512;
    const int es = (int)dtype_size(a.dtype);
    // widest row tile (<= 16 rows, power of two) whose transposed copy of X fits shared memory
    // beside a minimal staging area (two blocks per warp)
    int mt = 1;
    while (mt < 16 && (uint32_t)mt < a.M) mt *= 2;
    {
        const LaunchPlan &pw = w.plan_wide;
        const size_t min_stage_w = 256 + (size_t)(pw.threads / 32) * 2 * bb;
        while (mt > 1 && native_smem(w.K, mt * es, mt, pw.max_cols, pw.threads / 32) + min_stage_w > 200 * 1024) mt /= 2;
    }
    // A small tile leaves room for several CTAs per SM, whose stream and gather phases then
    // overlap (also across neighbouring calls); a tile of tens of KB gets the SM to itself.
    static const size_t wide_kb = (size_t)tuning_knob("SPTMM_WIDE_KB", 32);
    const bool wide = xs_bytes(w.K, mt * es) > wide_kb * 1024;
    const LaunchPlan &plan = wide ? w.plan_wide : w.plan;
    const uint32_t threads = plan.threads, nwarps = threads / 32;
    if (plan.grid > (uint32_t)kMaxGrid || nwarps > (uint32_t)kMaxWarps)
        return fail(SPTMM_ERR_INVALID, "internal: launch plan %u x %u out of range", plan.grid, threads);
    const size_t min_stage = 256 + (size_t)nwarps * 2 * bb;
    const size_t base_smem = native_smem(w.K, mt * es, mt, plan.max_cols, nwarps);
    const size_t gap = 1024;                  // dynamic shared memory before the tile's fixed address
    if (gap + base_smem + min_stage > 227 * 1024)
        return fail(SPTMM_ERR_UNSUPPORTED, "gemv: K=%u rows of %d-byte activations do not fit shared memory", w.K, es);

    // staging area: what a warp's slice holds beyond the registers, in one round if the budget
    // allows, else in double-buffered rounds of half the room each
    const uint32_t pd = delta ? 0u : (uint32_t)prefetch_depth(mt, wide);
    const uint32_t per_warp = (plan.max_cta_blocks + nwarps - 1) / nwarps + 1;
    const uint32_t need = per_warp > pd ? per_warp - pd : 0;
    // Beside a tile of more than 16 KB a smaller staging area pays: three such CTAs fit an SM instead
    // of two, so a neighbouring call's CTAs stream while this one gathers (6912x2560, 4 streams /
    // 1 stream: M=4 int8 6.1 -> 5.8 / 9.8 -> 8.5 us, M=1 fp32 5.9 -> 4.7 / 8.7 -> 7.6 us; the
    // one-row int8 tile wants the larger area: 3.35 against 3.5 us; 14 KB tiles are indifferent).
    static const size_t stage_big_kb = (size_t)tuning_knob("SPTMM_STAGE_BIG_KB", 30);
    const size_t stage_kb = xs_bytes(w.K, mt * es) > 16 * 1024 ? std::min((size_t)tune().smem_kb, stage_big_kb) : (size_t)tune().smem_kb;
    const size_t budget = wide ? (size_t)225 * 1024
                               : std::min(base_smem + std::max(stage_kb * 1024, min_stage), (size_t)225 * 1024);
    const uint32_t room = (uint32_t)((budget - base_smem - 256) / ((size_t)nwarps * bb));   // blocks per warp
    const uint32_t half = need == 0 ? 0 : (need <= room ? need : std::max(1u, room / 2));
    const uint32_t halves = need <= room ? 1 : 2;
    const size_t smem = gap + base_smem + 256 + (size_t)nwarps * halves * half * bb;

    NativeParams prm;
    prm.idx = (const uint4 *)a.arrays[0];
    prm.blk_off = (const uint32_t *)a.arrays[1];
    prm.X = a.X; prm.C = a.C;
#ifdef SPTMM_TUNING
    prm.trace = g_trace;
    prm.trace_ctas = (uint32_t)tuning_knob("SPTMM_TRACE_CTAS", 8);
#endif
    prm.status = a.status ? a.status : (uint32_t *)w.plan.d_status;
    prm.K = w.K; prm.N = w.N; prm.M = a.M;
    prm.max_cols = plan.max_cols;
    prm.x_colmajor = (a.flags & SPTMM_X_COLMAJOR) ? 1 : 0;
    prm.c_colmajor = (a.flags & SPTMM_C_COLMAJOR) ? 1 : 0;
    prm.uniform_nbl = w.uniform_nbl;
    prm.one = 1;
    prm.x_early = ((a.flags & SPTMM_LAUNCH_PDL) == 0 && tuning_knob("SPTMM_X_EARLY", 1)) ? 1 : 0;
    prm.n_peers = a.n_peers;
    for (uint32_t r = 0; r < 8; r++) {
        prm.Cp[r] = r < a.n_peers ? a.C_peers[r] : nullptr;
        prm.col_bound[r] = a.n_peers ? (uint32_t)((uint64_t)w.N * std::min(r, a.n_peers) / a.n_peers) : 0;
    }
    prm.col_bound[8] = a.n_peers ? w.N : 0;
    if (a.n_peers) prm.col_bound[a.n_peers] = w.N;
    prm.ldx = a.ldx ? a.ldx : w.K; prm.accumulate = a.accumulate ? 1u : 0u;
    prm.scaled = a.scaled ? 1u : 0u; prm.row_scale = a.row_scale; prm.out_scale = a.out_scale;
    prm.half_blocks = half;
    prm.stage_blocks = halves * half;
    prm.stage_off = (uint32_t)base_smem;
    for (uint32_t i = 0; i <= plan.grid; i++) { prm.cta_blk[i] = plan.cta_blk[i]; prm.cta_col[i] = plan.cta_col[i]; }
    const dim3 grid(plan.grid, (a.M + mt - 1) / mt, 1);
    const bool pdl = (a.flags & SPTMM_LAUNCH_PDL) != 0;
    cudaStream_t st = (cudaStream_t)a.stream;
    switch (a.dtype) {
        case SPTMM_I8:  return launch_dtype<SPTMM_I8>(prm, mt, (int)pd, wide, grid, threads, smem, pdl, st);
        case SPTMM_F16: return launch_dtype<SPTMM_F16>(prm, mt, (int)pd, wide, grid, threads, smem, pdl, st);
        case SPTMM_F32: return launch_dtype<SPTMM_F32>(prm, mt, (int)pd, wide, grid, threads, smem, pdl, st);
    }
    return fail(SPTMM_ERR_INVALID, "gemv: unknown dtype %u", a.dtype);
}

int launch_native_u16(const GemvArgs &a) { return launch_native(a, false); }
int launch_native_delta(const GemvArgs &a) { return launch_native(a, true); }

}  // namespace sptmm
