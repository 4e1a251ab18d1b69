// device_common.cuh -- device helpers shared by the kernels: activation traits, the
// transposed activation tile in shared memory, row gathers and warp reductions.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "internal.h"

namespace sptmm {

#define SPTMM_CUDA_TRY(expr)                                                            \
    do {                                                                                \
        cudaError_t e__ = (expr);                                                       \
        if (e__ != cudaSuccess)                                                         \
            return fail(SPTMM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

template <int DT> struct ActTraits;
template <> struct ActTraits<SPTMM_I8>  { using elem = int8_t; using acc = int32_t; static constexpr int size = 1; };
template <> struct ActTraits<SPTMM_F16> { using elem = __half; using acc = float;   static constexpr int size = 2; };
template <> struct ActTraits<SPTMM_F32> { using elem = float;  using acc = float;   static constexpr int size = 4; };

// Programmatic dependent launch: let the next kernel in the stream start its prologue now, and
// wait until the previous kernel has completed and its writes are visible.  Both are no-ops
// for a launch without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior_grid()   { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// The activation tile lives in shared memory TRANSPOSED: row k holds the MT values
// X[m0..m0+MT)[k] back to back (RB = MT*sizeof(elem) bytes), so one gather of row k feeds all
// MT accumulators.  Row K is an all-zero row: padded list entries carry index K.
template <int RB> struct RowWords { static constexpr int n = RB < 4 ? 1 : RB / 4; };

// The tile always starts at this absolute address of the CTA's shared window (dynamic shared
// memory starts at 1024 plus the kernel's static shared memory; kernels skip the gap).  With
// the base a compile-time constant, a gather is one shared load whose address is row*RB plus an
// immediate -- no add per gather.
constexpr uint32_t kXsAbs = 2048;

__device__ __forceinline__ unsigned char *tile_base(unsigned char *dyn_smem)
{
    return dyn_smem + (kXsAbs - (uint32_t)__cvta_generic_to_shared(dyn_smem));
}

// `off`: byte offset of the tile from the fixed address (0 for the kernels that have one tile; the
// compiler folds it away there)
template <int RB>
__device__ __forceinline__ void load_row(uint32_t row, uint32_t (&r)[RowWords<RB>::n], uint32_t off = 0)
{
    const uint32_t a = row * RB + off;
    if constexpr (RB == 1) asm volatile("ld.shared.s8 %0, [%1+2048];" : "=r"(r[0]) : "r"(a));
    else if constexpr (RB == 2) asm volatile("ld.shared.u16 %0, [%1+2048];" : "=r"(r[0]) : "r"(a));
    else if constexpr (RB == 4) asm volatile("ld.shared.u32 %0, [%1+2048];" : "=r"(r[0]) : "r"(a));
    else if constexpr (RB == 8) asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+2048];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
    else {
#pragma unroll
        for (int i = 0; i < RB / 16; i++)
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+2048];"
                         : "=r"(r[4 * i]), "=r"(r[4 * i + 1]), "=r"(r[4 * i + 2]), "=r"(r[4 * i + 3]) : "r"(a + 16 * i));
    }
}

template <int DT, int MT>
__device__ __forceinline__ void gather_add(typename ActTraits<DT>::acc (&acc)[MT], uint32_t row, uint32_t off = 0)
{
    constexpr int RB = MT * ActTraits<DT>::size;
    uint32_t r[RowWords<RB>::n];
    load_row<RB>(row, r, off);
    if constexpr (DT == SPTMM_I8 && MT == 1) {
        acc[0] += (int32_t)r[0];                                     // the load sign-extends
    } else if constexpr (DT == SPTMM_I8) {
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] += (int32_t)(int8_t)(r[m >> 2] >> (8 * (m & 3)));
    } else if constexpr (DT == SPTMM_F16) {
        // mixed-precision add (f32 += f16, one instruction, exact conversion, round to nearest)
        if constexpr (MT == 1) {
            asm("{ .reg .f16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.f32.f16 %0, lo, %0; }" : "+f"(acc[0]) : "r"(r[0]));
        } else {
#pragma unroll
            for (int m = 0; m < MT; m += 2)
                asm("{ .reg .f16 lo, hi; mov.b32 {lo, hi}, %2; add.rn.f32.f16 %0, lo, %0; add.rn.f32.f16 %1, hi, %1; }"
                    : "+f"(acc[m]), "+f"(acc[m + 1]) : "r"(r[m >> 1]));
        }
    } else {
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] += __uint_as_float(r[m]);
    }
}

__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c)     // a*b + c
{
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One lane's running sums over MT rows of X.  The generic form keeps one 32-bit sum per row and
// adds a gathered tile row element by element.
//
// For int8 tiles of two or more rows that costs a sign extension and an add per element, which
// makes instruction issue -- not memory -- the limit.  The packed form removes most of it: the
// tile then holds x+128 as unsigned bytes (`kBiased`; the zero row holds 128), a gathered word
// is split by two byte permutes into its even and odd bytes, each as two 16-bit fields of one
// register ({b0,0,b2,0} and {b1,0,b3,0}), and one 32-bit add per register accumulates two rows
// at once.  A 16-bit field holds 257 such bytes, so the caller announces its gathers with
// reserve() and the fields are spilled into the 32-bit sums (minus 128 per gather) every 256
// gathers at most.  Results are exact.
template <int DT, int MT, bool PACKED = (DT == SPTMM_I8 && MT > 1)>
struct LaneAcc {
    using acc_t = typename ActTraits<DT>::acc;
    static constexpr bool kBiased = false;
    acc_t v[MT];
    uint32_t off;                                  // byte offset of the tile read from (see load_row)
    __device__ __forceinline__ void clear(uint32_t /*one*/, uint32_t off_ = 0)
    {
        off = off_;
#pragma unroll
        for (int m = 0; m < MT; m++) v[m] = acc_t(0);
    }
    __device__ __forceinline__ void reserve(uint32_t) {}
    __device__ __forceinline__ void add(uint32_t row) { gather_add<DT, MT>(v, row, off); }
    __device__ __forceinline__ void finish() {}
};

template <int MT>
struct LaneAcc<SPTMM_I8, MT, true> {
    using acc_t = int32_t;
    static constexpr bool kBiased = true;
    static constexpr int NP = MT / 2;          // packed registers: MT=2 -> 1, else two per tile word
    int32_t v[MT];
    uint32_t pk[NP];
    uint32_t n;                                // gathers held in the 16-bit fields
    uint32_t one;                              // the value 1, unknown to the compiler (see add())
    uint32_t off;                              // byte offset of the tile read from (see load_row)
    __device__ __forceinline__ void clear(uint32_t one_, uint32_t off_ = 0)
    {
        one = one_; off = off_;
#pragma unroll
        for (int m = 0; m < MT; m++) v[m] = 0;
#pragma unroll
        for (int j = 0; j < NP; j++) pk[j] = 0;
        n = 0;
    }
    __device__ __forceinline__ void finish()
    {
        const int32_t bias = (int32_t)(128u * n);
        if constexpr (MT == 2) {
            v[0] += (int32_t)(pk[0] & 0xffffu) - bias;
            v[1] += (int32_t)(pk[0] >> 16) - bias;
        } else {
#pragma unroll
            for (int q = 0; q < MT / 4; q++) {
                v[4 * q + 0] += (int32_t)(pk[2 * q] & 0xffffu) - bias;
                v[4 * q + 2] += (int32_t)(pk[2 * q] >> 16) - bias;
                v[4 * q + 1] += (int32_t)(pk[2 * q + 1] & 0xffffu) - bias;
                v[4 * q + 3] += (int32_t)(pk[2 * q + 1] >> 16) - bias;
            }
        }
#pragma unroll
        for (int j = 0; j < NP; j++) pk[j] = 0;
        n = 0;
    }
    __device__ __forceinline__ void reserve(uint32_t gathers)      // warp-uniform
    {
        if (n + gathers > 256u) finish();
        n += gathers;
    }
    __device__ __forceinline__ void add(uint32_t row)
    {
        uint32_t r[RowWords<MT>::n];
        load_row<MT>(row, r, off);
        // The permutes run on the integer ALU pipe; plain adds would too, and with 16 rows that
        // pipe, not shared memory, bounds the kernel.  Written as multiply-adds by a 1 the
        // compiler cannot see through, the additions go to the FMA pipe instead and the two
        // pipes share the work.
        if constexpr (MT == 2) {
            pk[0] = mad_u32(__byte_perm(r[0], 0u, 0x4140), one, pk[0]);                  // {b0, 0, b1, 0}
        } else {
#pragma unroll
            for (int q = 0; q < MT / 4; q++) {
                pk[2 * q] = mad_u32(__byte_perm(r[q], 0u, 0x4240), one, pk[2 * q]);          // {b0, 0, b2, 0}
                pk[2 * q + 1] = mad_u32(__byte_perm(r[q], 0u, 0x4341), one, pk[2 * q + 1]);  // {b1, 0, b3, 0}
            }
        }
    }
};

__device__ __forceinline__ int32_t warp_sum(int32_t v) { return __reduce_add_sync(0xffffffffu, v); }

// Sum N values per lane over the 32 lanes of a warp so that the lanes end up holding DIFFERENT
// sums: each round exchanges half of the values with the lane `off` away and keeps the other half
// (a transposing butterfly: N/2 + N/4 + ... shuffles instead of N full reductions).  On return
// lane l holds the sum of value l / (32/N).
template <typename T, int N>
struct TransposeSum {
    static __device__ __forceinline__ T run(const T (&v)[N], uint32_t lane, uint32_t off)
    {
        T w[N / 2];
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < N / 2; i++) {
            const T send = up ? v[i] : v[i + N / 2];
            const T mine = up ? v[i + N / 2] : v[i];
            w[i] = mine + __shfl_xor_sync(0xffffffffu, send, off);
        }
        return TransposeSum<T, N / 2>::run(w, lane, off >> 1);
    }
};
template <typename T>
struct TransposeSum<T, 1> {
    static __device__ __forceinline__ T run(const T (&v)[1], uint32_t, uint32_t off)
    {
        T s = v[0];
        for (uint32_t o = off; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        return s;
    }
};

// Integer sums of finished lists on their way to the CTA's column sums in shared memory.  Adding a
// list's MT sums one by one (reduce over the warp, lane 0 adds, next row) is a chain of dependent
// steps that costs more than gathering a block; and MT full warp reductions keep the reduction unit
// busy for longer than the gathers of a short list take.  Here a list's sums are reduced by the
// transposing butterfly above (lane l ends with row l / (32/MT)), one lane per row parks its sum in
// a register, and when every lane is taken -- or the warp runs out of lists -- ONE atomic
// instruction adds up to 32 sums to their columns.
template <int MT>
struct PendingSums {
    static constexpr uint32_t kLists = 32 / MT;      // lists that fit the warp's lanes; also the lanes per row
    int keep;
    uint32_t at, pend;
    __device__ __forceinline__ void clear() { keep = 0; at = 0; pend = 0; }
    __device__ __forceinline__ void drain(int *c_s, uint32_t lane)
    {
        if ((lane & (kLists - 1)) < pend) atomicAdd(c_s + at, keep);
        pend = 0;
    }
    // every lane calls this with its partial sums of the list that just ended; v is zeroed
    __device__ __forceinline__ void push(int32_t (&v)[MT], uint32_t col, bool negative, int *c_s, uint32_t lane)
    {
        int s;
        if constexpr (MT == 1) s = __reduce_add_sync(0xffffffffu, v[0]);
        else s = TransposeSum<int, MT>::run(v, lane, 16);
        if ((lane & (kLists - 1)) == pend) { keep = negative ? -s : s; at = col * MT + lane / kLists; }
#pragma unroll
        for (int m = 0; m < MT; m++) v[m] = 0;
        if (++pend == kLists) drain(c_s, lane);
    }
};

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 4 x MT byte transpose in registers: w[m] holds bytes k0..k0+3 of row m; on return
// o[i*(MT/4) + j] is word j of tile row k0+i, i.e. the bytes of rows 4j..4j+3 at k0+i.
template <int MT>
__device__ __forceinline__ void transpose_bytes4(const uint32_t (&w)[MT], uint32_t (&o)[MT])
{
    static_assert(MT % 4 == 0, "row tiles of 4, 8 or 16");
#pragma unroll
    for (int j = 0; j < MT / 4; j++) {
        const uint32_t t0 = __byte_perm(w[4 * j], w[4 * j + 1], 0x5140);      // a0 b0 a1 b1
        const uint32_t t1 = __byte_perm(w[4 * j + 2], w[4 * j + 3], 0x5140);  // c0 d0 c1 d1
        const uint32_t t2 = __byte_perm(w[4 * j], w[4 * j + 1], 0x7362);      // a2 b2 a3 b3
        const uint32_t t3 = __byte_perm(w[4 * j + 2], w[4 * j + 3], 0x7362);  // c2 d2 c3 d3
        o[0 * (MT / 4) + j] = __byte_perm(t0, t1, 0x5410);
        o[1 * (MT / 4) + j] = __byte_perm(t0, t1, 0x7632);
        o[2 * (MT / 4) + j] = __byte_perm(t2, t3, 0x5410);
        o[3 * (MT / 4) + j] = __byte_perm(t2, t3, 0x7632);
    }
}

// Fill the transposed tile from X.  mv = valid rows of this tile (the rest read as zero).
// Lanes run along k so that global reads coalesce and shared writes spread over the banks.
// BIASED (int8 only): store x+128 as an unsigned byte, the form LaneAcc's packed sums expect.
template <int DT, int MT, bool BIASED = false>
__device__ __forceinline__ void stage_x(unsigned char *xs, const void *Xv, uint32_t K, uint32_t M,
                                        uint32_t m0, uint32_t mv, bool x_colmajor, uint32_t ldx = 0)
{
    // ldx: elements between rows of a row-major X (0 = K); a K-tile of a wider matrix passes the full width
    const size_t LD = ldx ? ldx : K;
    static_assert(!BIASED || DT == SPTMM_I8, "only int8 tiles are biased");
    using elem = typename ActTraits<DT>::elem;
    [[maybe_unused]] const auto biased = [](elem v) -> elem {
        if constexpr (BIASED) return (elem)((unsigned char)v ^ 0x80u);
        else return v;
    };
    constexpr int ES = ActTraits<DT>::size;
    elem *dst = reinterpret_cast<elem *>(xs);
    const elem *X = reinterpret_cast<const elem *>(Xv);
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    if (MT == 1 && !x_colmajor && ((reinterpret_cast<uintptr_t>(X + (size_t)m0 * LD) & 15) == 0)) {
        const uint32_t vec = (K * ES) / 16;
        const uint4 *src = reinterpret_cast<const uint4 *>(X + (size_t)m0 * LD);
        for (uint32_t i = tid; i < vec; i += nt) reinterpret_cast<uint4 *>(xs)[i] = __ldg(src + i);
        for (uint32_t k = vec * (16 / ES) + tid; k < K; k += nt) dst[k] = X[(size_t)m0 * LD + k];
    } else if (MT > 1 && !x_colmajor && (K % (4 / ES)) == 0 && (LD % (4 / ES)) == 0 && (reinterpret_cast<uintptr_t>(X) & 3) == 0) {
        // One thread takes one 32-bit word (KP = 4/ES consecutive k) from each of the MT rows --
        // coalesced along k -- transposes the MT x KP elements in registers and writes the KP
        // finished tile rows (MT*4 contiguous bytes) with vector stores.
        constexpr int KP = 4 / ES;
        const uint32_t pieces = K / KP;
        for (uint32_t pc = tid; pc < pieces; pc += nt) {
            uint32_t w[MT];
#pragma unroll
            for (int m = 0; m < MT; m++)
                w[m] = (uint32_t)m < mv ? __ldg(reinterpret_cast<const uint32_t *>(X + (size_t)(m0 + m) * LD) + pc) : 0u;
            uint32_t o[MT];                      // o[i*(MT/KP) + j]: word j of tile row k0+i
            if constexpr (ES == 4) {
#pragma unroll
                for (int m = 0; m < MT; m++) o[m] = w[m];
            } else if constexpr (ES == 2) {
#pragma unroll
                for (int j = 0; j < MT / 2; j++) {
                    o[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x5410);
                    o[MT / 2 + j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x7632);
                }
            } else {
                if constexpr (MT == 2) {
                    // rows k0..k0+3 hold two bytes each: (a_i, b_i)
                    o[0] = __byte_perm(w[0], w[1], 0x5140);          // a0 b0 a1 b1
                    o[1] = __byte_perm(w[0], w[1], 0x7362);          // a2 b2 a3 b3
                } else if constexpr (MT >= 4) {
                    transpose_bytes4<MT>(w, o);
                }
            }
            if constexpr (BIASED) {
#pragma unroll
                for (int m = 0; m < MT; m++) o[m] ^= 0x80808080u;
            }
            uint32_t *out = reinterpret_cast<uint32_t *>(xs + (size_t)pc * KP * MT * ES);   // MT words
            if constexpr (MT == 2) {
                *reinterpret_cast<uint2 *>(out) = make_uint2(o[0], o[1]);
            } else {
#pragma unroll
                for (int q = 0; q < MT / 4; q++)
                    reinterpret_cast<uint4 *>(out)[q] = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
            }
        }
    } else {
        for (uint32_t m = 0; m < (uint32_t)MT; m++) {
            if (m < mv) {
                for (uint32_t k = tid; k < K; k += nt)
                    dst[(size_t)k * MT + m] = biased(x_colmajor ? X[(size_t)k * M + m0 + m] : X[(size_t)(m0 + m) * LD + k]);
            } else {
                for (uint32_t k = tid; k < K; k += nt) dst[(size_t)k * MT + m] = biased(elem(0));
            }
        }
    }
    if (tid < (uint32_t)MT) dst[(size_t)K * MT + tid] = biased(elem(0));     // the zero row
}

__host__ __device__ inline size_t xs_bytes(uint32_t K, int rb) { return (((size_t)K + 1) * rb + 15) & ~(size_t)15; }

}  // namespace sptmm
