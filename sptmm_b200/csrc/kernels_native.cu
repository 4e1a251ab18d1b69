// kernels_native.cu -- the B200 kernel for the native u16 format (SPTMM_FMT_U16_V256).
//
// Work it replaces: rowWiseSplit3Small4 (main.cu:556-594), one 32-thread CTA per column with
// two-byte index loads and byte gathers through L1, re-streaming every index once per row of X.
//
// Design.  The encoded matrix is one contiguous run of 512-byte blocks (256 sorted row indices
// of one column and one sign, see host_encode.cpp).  The grid is one CTA per SM; a plan made at
// upload time gives CTA i a contiguous range of whole columns with an equal share of blocks,
// and inside the CTA each warp takes an equal contiguous slice of those blocks, so every warp
// streams one linear piece of memory with 16-byte loads per lane, P blocks in flight.
// The activation tile sits transposed in shared memory, so one gather serves MT rows of X and
// the index stream is read once for up to 16 rows.  Nothing is multiplied.
// A warp's slice can start and end inside a column: sums for its first and last column go to
// per-warp slots that are folded in warp order after a barrier, all other columns are owned by
// one warp, so results do not depend on scheduling (integer and floating point alike).
// With programmatic dependent launch the index prefetch is issued before the wait on the
// previous kernel, which hides launch latency and the DRAM ramp behind that kernel's tail.
#include "device_common.cuh"

namespace sptmm {

struct NativeParams {
    const uint4 *idx;            // total_blocks * 32 vectors
    const uint32_t *blk_off;     // 2N+1
    const CtaPlan *plan;         // grid entries
    const void *X;
    void *C;
    uint32_t K, N, M;
    uint32_t max_cols;
    uint32_t x_colmajor, c_colmajor, evict_first;
};

template <int DT, int MT, int P, int MINB>
__global__ void __launch_bounds__(512, MINB) k_u16_v256(const NativeParams p)
{
    using acc_t = typename ActTraits<DT>::acc;
    constexpr int RB = MT * ActTraits<DT>::size;
    extern __shared__ __align__(16) unsigned char smem[];

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const CtaPlan plan = p.plan[blockIdx.x];
    const uint32_t ncols = plan.c1 - plan.c0, nlists = 2 * ncols;
    const uint32_t nb = plan.b1 - plan.b0;
    const uint32_t wb0 = plan.b0 + (uint32_t)(((uint64_t)nb * warp) / nwarps);
    const uint32_t wb1 = plan.b0 + (uint32_t)(((uint64_t)nb * (warp + 1)) / nwarps);
    const uint64_t ef = p.evict_first ? l2_evict_first_policy() : 0ull;

    // ---- prefetch: weights do not depend on the previous kernel
    const uint4 *src = p.idx + (size_t)wb0 * 32 + lane;
    uint4 buf[P];
#pragma unroll
    for (int i = 0; i < P; i++)
        if (wb0 + i < wb1) buf[i] = ld_stream16(src + (size_t)i * 32, ef);

    pdl_launch_dependents();
    pdl_wait_prior_grid();

    // ---- shared memory carve-up
    unsigned char *xs = smem;
    uint32_t *off_s = reinterpret_cast<uint32_t *>(smem + xs_bytes(p.K, RB));      // nlists+1
    acc_t *c_s = reinterpret_cast<acc_t *>(off_s + 2 * p.max_cols + 1 + ((2 * p.max_cols + 1) & 1));
    acc_t *head_s = c_s + (size_t)p.max_cols * MT;                                  // nwarps*MT
    acc_t *tail_s = head_s + (size_t)nwarps * MT;                                   // nwarps*MT
    uint32_t *hcol_s = reinterpret_cast<uint32_t *>(tail_s + (size_t)nwarps * MT);  // nwarps
    uint32_t *tcol_s = hcol_s + nwarps;

    const uint32_t m0 = blockIdx.y * MT;
    const uint32_t mv = min((uint32_t)MT, p.M - m0);
    stage_x<DT, MT>(xs, p.X, p.K, p.M, m0, mv, p.x_colmajor != 0);
    for (uint32_t i = threadIdx.x; i <= nlists; i += blockDim.x) off_s[i] = p.blk_off[2 * plan.c0 + i];
    for (uint32_t i = threadIdx.x; i < ncols * MT; i += blockDim.x) c_s[i] = acc_t(0);
    for (uint32_t i = threadIdx.x; i < nwarps * MT; i += blockDim.x) { head_s[i] = acc_t(0); tail_s[i] = acc_t(0); }
    __syncthreads();

    if (wb0 < wb1) {
        // list that holds block wb0 / block wb1-1: count boundaries at or below the block
        uint32_t li = 0, llast = 0;
        for (uint32_t r = 1; r <= nlists; r += 32) {          // warp-uniform trip count
            const uint32_t i = r + lane;
            const uint32_t o = i <= nlists ? off_s[i] : 0xffffffffu;
            li += __popc(__ballot_sync(0xffffffffu, o <= wb0));
            llast += __popc(__ballot_sync(0xffffffffu, o <= wb1 - 1));
        }
        const uint32_t first_col = li >> 1, last_col = llast >> 1;
        if (lane == 0) { hcol_s[warp] = first_col; tcol_s[warp] = last_col; }

        acc_t acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = acc_t(0);
        uint32_t bound = off_s[li + 1];
        bool dirty = false;

        auto flush = [&]() {
            const uint32_t col = li >> 1;
            acc_t *dst = col == first_col ? head_s + warp * MT : (col == last_col ? tail_s + warp * MT : c_s + col * MT);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                acc_t v = warp_sum(acc[m]);
                if (lane == 0) dst[m] += (li & 1) ? -v : v;
                acc[m] = acc_t(0);
            }
        };

        for (uint32_t base = wb0; base < wb1; base += P) {
#pragma unroll
            for (int i = 0; i < P; i++) {
                const uint32_t b = base + i;
                if (b < wb1) {
                    const uint4 v = buf[i];
                    if (b + P < wb1) buf[i] = ld_stream16(src + (size_t)(b + P - wb0) * 32, ef);
                    while (b >= bound) {
                        if (dirty) { flush(); dirty = false; }
                        li++;
                        bound = off_s[li + 1];
                    }
                    dirty = true;
                    gather_add<DT, MT>(acc, xs, v.x & 0xffffu);
                    gather_add<DT, MT>(acc, xs, v.x >> 16);
                    gather_add<DT, MT>(acc, xs, v.y & 0xffffu);
                    gather_add<DT, MT>(acc, xs, v.y >> 16);
                    gather_add<DT, MT>(acc, xs, v.z & 0xffffu);
                    gather_add<DT, MT>(acc, xs, v.z >> 16);
                    gather_add<DT, MT>(acc, xs, v.w & 0xffffu);
                    gather_add<DT, MT>(acc, xs, v.w >> 16);
                }
            }
        }
        if (dirty) flush();
    } else if (lane == 0) {
        hcol_s[warp] = 0xffffffffu; tcol_s[warp] = 0xffffffffu;
    }
    __syncthreads();

    // ---- fold the per-warp edge sums in warp order (one thread per row of the tile)
    if (threadIdx.x < (uint32_t)MT) {
        const uint32_t m = threadIdx.x;
        for (uint32_t w = 0; w < nwarps; w++) {
            const uint32_t hc = hcol_s[w], tc = tcol_s[w];
            if (hc != 0xffffffffu) {
                c_s[hc * MT + m] += head_s[w * MT + m];
                if (tc != hc) c_s[tc * MT + m] += tail_s[w * MT + m];
            }
        }
    }
    __syncthreads();

    acc_t *C = reinterpret_cast<acc_t *>(p.C);
    for (uint32_t i = threadIdx.x; i < ncols * mv; i += blockDim.x) {
        const uint32_t m = i / ncols, col = i - m * ncols;
        const size_t o = p.c_colmajor ? (size_t)(plan.c0 + col) * p.M + m0 + m : (size_t)(m0 + m) * p.N + plan.c0 + col;
        C[o] = c_s[col * MT + m];
    }
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
    return s;
}

template <int DT, int MT, int P, int MINB>
static int launch_one(const NativeParams &prm, dim3 grid, uint32_t threads, size_t smem, bool pdl, cudaStream_t st)
{
    static int configured_device = -1;
    int dev = 0;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (configured_device != dev) {
        SPTMM_CUDA_TRY(cudaFuncSetAttribute(k_u16_v256<DT, MT, P, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured_device = dev;
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

template <int DT>
static int launch_dtype(const NativeParams &prm, int mt, dim3 grid, uint32_t threads, size_t smem, bool pdl,
                        cudaStream_t st, int prefetch)
{
    switch (mt) {
        case 1:
            if (prefetch >= 16) return launch_one<DT, 1, 16, 1>(prm, grid, threads, smem, pdl, st);
            if (prefetch <= 4) return launch_one<DT, 1, 4, 2>(prm, grid, threads, smem, pdl, st);
            return launch_one<DT, 1, 8, 2>(prm, grid, threads, smem, pdl, st);
        case 2: return launch_one<DT, 2, 8, 2>(prm, grid, threads, smem, pdl, st);
        case 4: return launch_one<DT, 4, 8, 2>(prm, grid, threads, smem, pdl, st);
        case 8: return launch_one<DT, 8, 4, 1>(prm, grid, threads, smem, pdl, st);
        case 16: return launch_one<DT, 16, 4, 1>(prm, grid, threads, smem, pdl, st);
    }
    return fail(SPTMM_ERR_INVALID, "internal: row tile %d", mt);
}

int launch_native_u16(const GemvArgs &a)
{
    const sptmm_weights &w = *a.w;
    const int es = (int)dtype_size(a.dtype);
    const uint32_t threads = w.plan.threads, nwarps = threads / 32;
    // widest row tile (<= 16 rows, power of two) whose transposed copy of X fits shared memory
    int mt = 1;
    while (mt < 16 && (uint32_t)mt < a.M) mt *= 2;
    const size_t cap = 200 * 1024;
    while (mt > 1 && native_smem(w.K, mt * es, mt, w.plan.max_cols, nwarps) > cap) mt /= 2;
    const size_t smem = native_smem(w.K, mt * es, mt, w.plan.max_cols, nwarps);
    if (smem > 227 * 1024)
        return fail(SPTMM_ERR_UNSUPPORTED, "gemv: K=%u rows of %d-byte activations do not fit shared memory", w.K, es);

    NativeParams prm;
    prm.idx = (const uint4 *)a.arrays[0];
    prm.blk_off = (const uint32_t *)a.arrays[1];
    prm.plan = (const CtaPlan *)w.plan.d_ctas;
    prm.X = a.X; prm.C = a.C;
    prm.K = w.K; prm.N = w.N; prm.M = a.M;
    prm.max_cols = w.plan.max_cols;
    prm.x_colmajor = (a.flags & SPTMM_X_COLMAJOR) ? 1 : 0;
    prm.c_colmajor = (a.flags & SPTMM_C_COLMAJOR) ? 1 : 0;
    prm.evict_first = tune().evict_first;
    const dim3 grid(w.plan.grid, (a.M + mt - 1) / mt, 1);
    const bool pdl = (a.flags & SPTMM_LAUNCH_PDL) != 0;
    cudaStream_t st = (cudaStream_t)a.stream;
    switch (a.dtype) {
        case SPTMM_I8:  return launch_dtype<SPTMM_I8>(prm, mt, grid, threads, smem, pdl, st, tune().prefetch);
        case SPTMM_F16: return launch_dtype<SPTMM_F16>(prm, mt, grid, threads, smem, pdl, st, tune().prefetch);
        case SPTMM_F32: return launch_dtype<SPTMM_F32>(prm, mt, grid, threads, smem, pdl, st, tune().prefetch);
    }
    return fail(SPTMM_ERR_INVALID, "gemv: unknown dtype %u", a.dtype);
}

int launch_native_delta(const GemvArgs &)
{
    return fail(SPTMM_ERR_UNSUPPORTED, "gemv: lane-delta format is not built yet");
}

}  // namespace sptmm
