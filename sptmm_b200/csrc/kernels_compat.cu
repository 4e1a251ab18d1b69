// kernels_compat.cu -- kernels that consume the reference's own encoded layouts byte-for-byte,
// plus the 2-bit comparator.
//
//  k_div       W_map_{8,16,32}_div, u16 [chunk][column][split]        (replaces main.cu:556-594)
//  k_delta256  W_map_delta2_div256, u8 gaps [block][column][256]      (replaces main.cu:599-764)
//  k_i2s       2-bit codes, 16 rows per word                          (replaces bitnet_kernels.cuh:75-111)
//  k_i2s_row   the same for one row of X with its activations in registers
//
// Differences from the reference kernels: multi-warp CTAs that stage the activation tile
// (transposed, up to 16 rows) in shared memory once, so the index stream is read once for all
// rows instead of once per row; gathers hit shared memory instead of L1; any shape is accepted
// at run time instead of a compile-time whitelist.
#include <atomic>

#include "device_common.cuh"

namespace sptmm {

// --------------------------------------------------------------------------------------------
struct DivParams {
    const uint16_t *wp, *wn;
    const void *X; void *C;
    uint32_t K, N, M, chunks;
    uint32_t x_colmajor, c_colmajor;
};

template <int DT, int MT, int SPLIT>
__global__ void __launch_bounds__(256) k_div(const DivParams p)
{
    using acc_t = typename ActTraits<DT>::acc;
    constexpr int CPW = 32 / SPLIT;              // columns a warp handles at once
    constexpr int U = 8;                         // chunks in flight
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const uint32_t m0 = blockIdx.y * MT, mv = min((uint32_t)MT, p.M - m0);
    stage_x<DT, MT>(tile_base(smem), p.X, p.K, p.M, m0, mv, p.x_colmajor != 0);
    __syncthreads();

    const uint32_t ngroups = p.N / CPW;
    const size_t stride = (size_t)SPLIT * p.N;   // elements between consecutive chunks
    acc_t *C = reinterpret_cast<acc_t *>(p.C);
    for (uint32_t g = blockIdx.x * nwarps + warp; g < ngroups; g += gridDim.x * nwarps) {
        const uint16_t *bp = p.wp + (size_t)g * 32 + lane;
        const uint16_t *bn = p.wn + (size_t)g * 32 + lane;
        acc_t ap[MT], an[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) { ap[m] = acc_t(0); an[m] = acc_t(0); }
        uint32_t j = 0;
        for (; j + U <= p.chunks; j += U) {
            uint16_t ip[U], in[U];
#pragma unroll
            for (int u = 0; u < U; u++) { ip[u] = __ldg(bp + (j + u) * stride); in[u] = __ldg(bn + (j + u) * stride); }
            // a caller-built layout may hold anything: an index past K reads the zero row, not beyond the tile
#pragma unroll
            for (int u = 0; u < U; u++) { gather_add<DT, MT>(ap, min((uint32_t)ip[u], p.K)); gather_add<DT, MT>(an, min((uint32_t)in[u], p.K)); }
        }
        for (; j < p.chunks; j++) {
            gather_add<DT, MT>(ap, min((uint32_t)__ldg(bp + j * stride), p.K));
            gather_add<DT, MT>(an, min((uint32_t)__ldg(bn + j * stride), p.K));
        }
        const uint32_t col = g * CPW + lane / SPLIT;
#pragma unroll
        for (int m = 0; m < MT; m++) {
            acc_t v = ap[m] - an[m];
#pragma unroll
            for (int o = SPLIT / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((lane % SPLIT) == 0 && (uint32_t)m < mv) {
                const size_t o = p.c_colmajor ? (size_t)col * p.M + m0 + m : (size_t)(m0 + m) * p.N + col;
                C[o] = v;
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
struct DeltaParams {
    const uint8_t *dp, *dn;
    const void *X; void *C;
    uint32_t K, N, M, half;      // half = S/2 entries per sign
    uint32_t x_colmajor, c_colmajor;
};

// One warp per column.  Lane l owns gaps 8l..8l+7 of each 256-entry block (one 8-byte load per
// sign); it sums them locally, one packed warp scan per block gives each lane its starting
// offset, and the running index is carried from block to block in 16-bit arithmetic exactly as
// the reference carries it (main.cu:650-665).  Entries past S/2 contribute nothing
// (main.cu:735).  The reference does eight warp scans per block; this does one.
template <int DT, int MT>
__global__ void __launch_bounds__(256) k_delta256(const DeltaParams p)
{
    using acc_t = typename ActTraits<DT>::acc;
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const uint32_t m0 = blockIdx.y * MT, mv = min((uint32_t)MT, p.M - m0);
    stage_x<DT, MT>(tile_base(smem), p.X, p.K, p.M, m0, mv, p.x_colmajor != 0);
    __syncthreads();

    const uint32_t nblk = (p.half + 255) / 256;
    const size_t bstride = (size_t)256 * p.N;
    acc_t *C = reinterpret_cast<acc_t *>(p.C);
    for (uint32_t col = blockIdx.x * nwarps + warp; col < p.N; col += gridDim.x * nwarps) {
        const uint8_t *bp = p.dp + (size_t)col * 256 + lane * 8;
        const uint8_t *bn = p.dn + (size_t)col * 256 + lane * 8;
        acc_t ap[MT], an[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) { ap[m] = acc_t(0); an[m] = acc_t(0); }
        uint32_t carry_p = 0, carry_n = 0;
        uint2 gp = make_uint2(0, 0), gn = make_uint2(0, 0);
        if (lane * 8 < p.half) {
            gp = __ldg(reinterpret_cast<const uint2 *>(bp));
            gn = __ldg(reinterpret_cast<const uint2 *>(bn));
        }
        for (uint32_t blk = 0; blk < nblk; blk++) {
            const uint2 cp = gp, cn = gn;
            const uint32_t e0 = blk * 256 + lane * 8;
            if (blk + 1 < nblk && e0 + 256 < p.half) {
                gp = __ldg(reinterpret_cast<const uint2 *>(bp + (blk + 1) * bstride));
                gn = __ldg(reinterpret_cast<const uint2 *>(bn + (blk + 1) * bstride));
            }
            uint32_t sp[8], sn[8], rp = 0, rn = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const bool valid = e0 + i < p.half;
                const uint32_t wpv = i < 4 ? cp.x : cp.y, wnv = i < 4 ? cn.x : cn.y;
                rp += valid ? (wpv >> (8 * (i & 3))) & 0xffu : 0u;
                rn += valid ? (wnv >> (8 * (i & 3))) & 0xffu : 0u;
                sp[i] = rp; sn[i] = rn;
            }
            uint32_t incl = (rn << 16) | rp;            // both fields stay below 65536 across 32 lanes
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= (uint32_t)o) incl += t;
            }
            const uint32_t excl = incl - ((rn << 16) | rp);
            const uint32_t base_p = carry_p + (excl & 0xffffu), base_n = carry_n + (excl >> 16);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const bool valid = e0 + i < p.half;
                const uint32_t ip = (base_p + sp[i]) & 0xffffu, in = (base_n + sn[i]) & 0xffffu;
                gather_add<DT, MT>(ap, (valid && ip < p.K) ? ip : p.K);
                gather_add<DT, MT>(an, (valid && in < p.K) ? in : p.K);
            }
            const uint32_t tot = __shfl_sync(0xffffffffu, incl, 31);
            carry_p = (carry_p + (tot & 0xffffu)) & 0xffffu;
            carry_n = (carry_n + (tot >> 16)) & 0xffffu;
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const acc_t v = warp_sum(ap[m] - an[m]);
            if (lane == 0 && (uint32_t)m < mv) {
                const size_t o = p.c_colmajor ? (size_t)col * p.M + m0 + m : (size_t)(m0 + m) * p.N + col;
                C[o] = v;
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
struct I2sParams {
    const uint32_t *w;           // [N][K/16]
    const int8_t *X; int32_t *C;
    uint32_t K, N, M;
    uint32_t x_colmajor, c_colmajor;
};

// Comparator.  Eight lanes share a column and split K; a word's 16 codes c = w+2 are isolated
// four at a time with a shift and a mask and fed to dp4a against four activations; the bias is
// removed once per output: sum (c-2) x = sum c x - 2 sum x.
template <int MT>
__global__ void __launch_bounds__(256) k_i2s(const I2sParams p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    int8_t *xs = reinterpret_cast<int8_t *>(smem);                       // [MT][K], row-major
    int32_t *sumx = reinterpret_cast<int32_t *>(smem + (((size_t)MT * p.K + 15) & ~(size_t)15));
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const uint32_t m0 = blockIdx.y * MT, mv = min((uint32_t)MT, p.M - m0);
    if (threadIdx.x < (uint32_t)MT) sumx[threadIdx.x] = 0;
    for (uint32_t m = 0; m < (uint32_t)MT; m++)
        for (uint32_t k = threadIdx.x; k < p.K; k += blockDim.x)
            xs[(size_t)m * p.K + k] = m < mv ? (p.x_colmajor ? p.X[(size_t)k * p.M + m0 + m] : p.X[(size_t)(m0 + m) * p.K + k]) : (int8_t)0;
    __syncthreads();
    for (uint32_t m = 0; m < (uint32_t)MT; m++) {
        int32_t s = 0;
        for (uint32_t k = threadIdx.x; k < p.K; k += blockDim.x) s += xs[(size_t)m * p.K + k];
        s = warp_sum(s);
        if (lane == 0) atomicAdd(&sumx[m], s);
    }
    __syncthreads();

    const uint32_t words = p.K / 16, q = lane >> 3, r = lane & 7;
    for (uint32_t c4 = (blockIdx.x * nwarps + warp) * 4; c4 < p.N; c4 += gridDim.x * nwarps * 4) {
        const uint32_t col = c4 + q;
        int32_t acc[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] = 0;
        if (col < p.N) {
            const uint32_t *wc = p.w + (size_t)col * words;
            for (uint32_t j = r; j < words; j += 8) {
                const uint32_t word = __ldg(wc + j);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int codes = (int)((word >> (2 * i)) & 0x03030303u);
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const int xv = *reinterpret_cast<const int *>(xs + (size_t)m * p.K + 16 * j + 4 * i);
                        acc[m] = __dp4a(xv, codes, acc[m]);
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
            int32_t v = acc[m];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            if (r == 0 && col < p.N && (uint32_t)m < mv) {
                const size_t o = p.c_colmajor ? (size_t)col * p.M + m0 + m : (size_t)(m0 + m) * p.N + col;
                p.C[o] = v - 2 * sumx[m];
            }
        }
    }
}

// One row of X (M = 1), K a multiple of 64 and at most NV*2048: a warp owns whole columns and reads a
// column's codes with full-width 16-byte loads (lane l takes vectors l, l+32, ...).  Since a lane
// meets the same rows of X in every column, its 64 bytes of X per vector stay in registers: no
// shared memory, no CTA barrier, and the next column's loads are in flight while this one is summed.
template <int NV>
__global__ void __launch_bounds__(128) k_i2s_row(const I2sParams p)
{
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint32_t tw = gridDim.x * nwarps, nvec = p.K / 64;
    uint32_t col = blockIdx.x * nwarps + warp;
    const uint4 *w4 = reinterpret_cast<const uint4 *>(p.w);
    pdl_launch_dependents();
    uint4 nxt[NV];
    auto load_col = [&](uint32_t c) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const uint32_t v = lane + 32u * i;
            nxt[i] = (c < p.N && v < nvec) ? __ldg(w4 + (size_t)c * nvec + v) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    load_col(col);                           // the weights do not depend on the kernel before
    pdl_wait_prior_grid();
    uint4 x[NV][4];
    int sumx = 0;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const uint32_t v = lane + 32u * i;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            x[i][w] = v < nvec ? __ldg(reinterpret_cast<const uint4 *>(p.X) + (size_t)v * 4 + w) : make_uint4(0u, 0u, 0u, 0u);
            sumx = __dp4a((int)x[i][w].x, 0x01010101, sumx);
            sumx = __dp4a((int)x[i][w].y, 0x01010101, sumx);
            sumx = __dp4a((int)x[i][w].z, 0x01010101, sumx);
            sumx = __dp4a((int)x[i][w].w, 0x01010101, sumx);
        }
    }
    sumx = warp_sum(sumx);
    for (; col < p.N; col += tw) {
        uint4 cur[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) cur[i] = nxt[i];
        load_col(col + tw);
        int acc = 0;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const uint32_t word[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
                acc = __dp4a((int)x[i][w].x, (int)(word[w] & 0x03030303u), acc);
                acc = __dp4a((int)x[i][w].y, (int)((word[w] >> 2) & 0x03030303u), acc);
                acc = __dp4a((int)x[i][w].z, (int)((word[w] >> 4) & 0x03030303u), acc);
                acc = __dp4a((int)x[i][w].w, (int)((word[w] >> 6) & 0x03030303u), acc);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) p.C[col] = acc - 2 * sumx;
    }
}

// --------------------------------------------------------------------------------------------
template <auto kern, typename Prm>
static int launch_generic(const Prm &prm, dim3 grid, size_t smem, bool pdl, cudaStream_t st, uint32_t threads = 256)
{
    if (smem > 48 * 1024) {          // opt in to large dynamic shared memory once per kernel and device
        static std::atomic<int> configured_device{-1};     // one instance per kernel (the kernel is a template argument)
        int dev = 0;
        SPTMM_CUDA_TRY(cudaGetDevice(&dev));
        if (configured_device.load(std::memory_order_acquire) != dev) {
            SPTMM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            configured_device.store(dev, std::memory_order_release);
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    SPTMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, prm));
    return SPTMM_OK;
}

static int pick_row_tile(uint32_t M, uint32_t K, int es, int max_mt)
{
    int mt = 1;
    while (mt < max_mt && (uint32_t)mt < M) mt *= 2;
    while (mt > 1 && xs_bytes(K, mt * es) > 160 * 1024) mt /= 2;
    return mt;
}

template <int DT, int SPLIT>
static int launch_div_mt(const DivParams &prm, int mt, dim3 grid, size_t smem, bool pdl, cudaStream_t st)
{
    switch (mt) {
        case 1: return launch_generic<k_div<DT, 1, SPLIT>>(prm, grid, smem, pdl, st);
        case 2: return launch_generic<k_div<DT, 2, SPLIT>>(prm, grid, smem, pdl, st);
        case 4: return launch_generic<k_div<DT, 4, SPLIT>>(prm, grid, smem, pdl, st);
        case 8: return launch_generic<k_div<DT, 8, SPLIT>>(prm, grid, smem, pdl, st);
    }
    return fail(SPTMM_ERR_INVALID, "internal: row tile %d", mt);
}

template <int DT>
static int launch_div_split(const DivParams &prm, uint32_t split, int mt, dim3 grid, size_t smem, bool pdl, cudaStream_t st)
{
    switch (split) {
        case 8:  return launch_div_mt<DT, 8>(prm, mt, grid, smem, pdl, st);
        case 16: return launch_div_mt<DT, 16>(prm, mt, grid, smem, pdl, st);
        case 32: return launch_div_mt<DT, 32>(prm, mt, grid, smem, pdl, st);
    }
    return fail(SPTMM_ERR_INVALID, "Wrong split size");     // the reference's message, main.cu:1039
}

int launch_div(const void *X, const uint16_t *wp, const uint16_t *wn, void *C, uint32_t dtype,
               uint32_t M, uint32_t K, uint32_t N, uint32_t S, uint32_t split, uint32_t flags, void *stream)
{
    if (!X || !wp || !wn || !C) return fail(SPTMM_ERR_INVALID, "row_split3_small: null pointer");
    if (split != 8 && split != 16 && split != 32) return fail(SPTMM_ERR_INVALID, "Wrong split size");
    if (M == 0 || K == 0 || N == 0 || K > 65535) return fail(SPTMM_ERR_INVALID, "row_split3_small: bad shape M=%u K=%u N=%u", M, K, N);
    if ((S & 1) || (S / 2) % split) return fail(SPTMM_ERR_INVALID, "row_split3_small: S/2=%u must be a multiple of split=%u", S / 2, split);
    if (N % (32 / split)) return fail(SPTMM_ERR_INVALID, "row_split3_small: N=%u must be a multiple of %u", N, 32 / split);
    const int es = (int)dtype_size(dtype), mt = pick_row_tile(M, K, es, 8);
    const size_t smem = xs_bytes(K, mt * es) + 1024;      // room to start the tile at its fixed address
    if (smem > 227 * 1024) return fail(SPTMM_ERR_UNSUPPORTED, "row_split3_small: K=%u does not fit shared memory", K);
    DivParams prm{wp, wn, X, C, K, N, M, (S / 2) / split, (flags & SPTMM_X_COLMAJOR) ? 1u : 0u, (flags & SPTMM_C_COLMAJOR) ? 1u : 0u};
    const uint32_t ngroups = N / (32 / split);
    const dim3 grid((ngroups + 7) / 8, (M + mt - 1) / mt, 1);
    const bool pdl = (flags & SPTMM_LAUNCH_PDL) != 0;
    switch (dtype) {
        case SPTMM_I8:  return launch_div_split<SPTMM_I8>(prm, split, mt, grid, smem, pdl, (cudaStream_t)stream);
        case SPTMM_F16: return launch_div_split<SPTMM_F16>(prm, split, mt, grid, smem, pdl, (cudaStream_t)stream);
        case SPTMM_F32: return launch_div_split<SPTMM_F32>(prm, split, mt, grid, smem, pdl, (cudaStream_t)stream);
    }
    return fail(SPTMM_ERR_INVALID, "unknown dtype %u", dtype);
}

template <int DT>
static int launch_delta_mt(const DeltaParams &prm, int mt, dim3 grid, size_t smem, bool pdl, cudaStream_t st)
{
    switch (mt) {
        case 1: return launch_generic<k_delta256<DT, 1>>(prm, grid, smem, pdl, st);
        case 2: return launch_generic<k_delta256<DT, 2>>(prm, grid, smem, pdl, st);
        case 4: return launch_generic<k_delta256<DT, 4>>(prm, grid, smem, pdl, st);
        case 8: return launch_generic<k_delta256<DT, 8>>(prm, grid, smem, pdl, st);
    }
    return fail(SPTMM_ERR_INVALID, "internal: row tile %d", mt);
}

int launch_delta256(const void *X, const uint8_t *dp, const uint8_t *dn, void *C, uint32_t dtype,
                    uint32_t M, uint32_t K, uint32_t N, uint32_t S, uint32_t flags, void *stream)
{
    if (!X || !dp || !dn || !C) return fail(SPTMM_ERR_INVALID, "row_split_delta2: null pointer");
    if (M == 0 || K == 0 || N == 0 || K > 65535) return fail(SPTMM_ERR_INVALID, "row_split_delta2: bad shape M=%u K=%u N=%u", M, K, N);
    if ((S & 1) || S == 0) return fail(SPTMM_ERR_INVALID, "row_split_delta2: S=%u must be even and non-zero", S);
    if ((reinterpret_cast<uintptr_t>(dp) | reinterpret_cast<uintptr_t>(dn)) & 7)
        return fail(SPTMM_ERR_INVALID, "row_split_delta2: gap arrays must be 8-byte aligned");
    const int es = (int)dtype_size(dtype), mt = pick_row_tile(M, K, es, 8);
    const size_t smem = xs_bytes(K, mt * es) + 1024;      // room to start the tile at its fixed address
    if (smem > 227 * 1024) return fail(SPTMM_ERR_UNSUPPORTED, "row_split_delta2: K=%u does not fit shared memory", K);
    DeltaParams prm{dp, dn, X, C, K, N, M, S / 2, (flags & SPTMM_X_COLMAJOR) ? 1u : 0u, (flags & SPTMM_C_COLMAJOR) ? 1u : 0u};
    const dim3 grid((N + 7) / 8, (M + mt - 1) / mt, 1);
    const bool pdl = (flags & SPTMM_LAUNCH_PDL) != 0;
    switch (dtype) {
        case SPTMM_I8:  return launch_delta_mt<SPTMM_I8>(prm, mt, grid, smem, pdl, (cudaStream_t)stream);
        case SPTMM_F16: return launch_delta_mt<SPTMM_F16>(prm, mt, grid, smem, pdl, (cudaStream_t)stream);
        case SPTMM_F32: return launch_delta_mt<SPTMM_F32>(prm, mt, grid, smem, pdl, (cudaStream_t)stream);
    }
    return fail(SPTMM_ERR_INVALID, "unknown dtype %u", dtype);
}

int launch_i2s(const GemvArgs &a)
{
    const sptmm_weights &w = *a.w;
    if (a.dtype != SPTMM_I8) return fail(SPTMM_ERR_UNSUPPORTED, "i2s comparator takes int8 activations only");
    int mt = 1;
    while (mt < 8 && (uint32_t)mt < a.M) mt *= 2;
    while (mt > 1 && (size_t)mt * w.K > 160 * 1024) mt /= 2;
    const size_t smem = (((size_t)mt * w.K + 15) & ~(size_t)15) + 64;
    if (smem > 227 * 1024) return fail(SPTMM_ERR_UNSUPPORTED, "i2s: K=%u does not fit shared memory", w.K);
    I2sParams prm{(const uint32_t *)a.arrays[0], (const int8_t *)a.X, (int32_t *)a.C, w.K, w.N, a.M,
                  (a.flags & SPTMM_X_COLMAJOR) ? 1u : 0u, (a.flags & SPTMM_C_COLMAJOR) ? 1u : 0u};
    const bool pdl = (a.flags & SPTMM_LAUNCH_PDL) != 0;
    cudaStream_t st = (cudaStream_t)a.stream;
    // One row, K a multiple of 64 up to 8192, X on a 16-byte boundary: the register form, a warp per
    // column, four warps per CTA and about four columns per warp (X is fetched once per warp).
    if (a.M == 1 && w.K % 64 == 0 && w.K <= 8192 && (reinterpret_cast<uintptr_t>(a.X) & 15) == 0) {
        const uint32_t sms = w.sm_count ? w.sm_count : 148u;
        const dim3 grid(std::max(1u, std::min((w.N + 15) / 16, 4 * sms)), 1, 1);
        const uint32_t nv = (w.K / 64 + 31) / 32;
        switch (nv) {
            case 1: return launch_generic<k_i2s_row<1>>(prm, grid, 0, pdl, st, 128);
            case 2: return launch_generic<k_i2s_row<2>>(prm, grid, 0, pdl, st, 128);
            case 3: return launch_generic<k_i2s_row<3>>(prm, grid, 0, pdl, st, 128);
            default: return launch_generic<k_i2s_row<4>>(prm, grid, 0, pdl, st, 128);
        }
    }
    // Otherwise four columns per warp, eight lanes per column, X in shared memory.
    const uint32_t threads = 256u, cols_per_cta = threads / 8;
    const dim3 grid((w.N + cols_per_cta - 1) / cols_per_cta, (a.M + mt - 1) / mt, 1);
    switch (mt) {
        case 1: return launch_generic<k_i2s<1>>(prm, grid, smem, pdl, st, threads);
        case 2: return launch_generic<k_i2s<2>>(prm, grid, smem, pdl, st, threads);
        case 4: return launch_generic<k_i2s<4>>(prm, grid, smem, pdl, st, threads);
        case 8: return launch_generic<k_i2s<8>>(prm, grid, smem, pdl, st, threads);
    }
    return fail(SPTMM_ERR_INVALID, "internal: row tile %d", mt);
}

}  // namespace sptmm
