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

// 16-byte streaming load that bypasses L1; with `policy` != 0 the line is also marked
// evict-first in L2 (weights are read once per matmul).
__device__ __forceinline__ uint64_t l2_evict_first_policy()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ uint4 ld_stream16(const uint4 *p, uint64_t policy)
{
    uint4 v;
    if (policy)
        asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
    else
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// The activation tile lives in shared memory TRANSPOSED: row k holds the MT values
// X[m0..m0+MT)[k] back to back (RB = MT*sizeof(elem) bytes), so one gather of row k feeds all
// MT accumulators.  Row K is an all-zero row: padded list entries carry index K.
template <int RB> struct RowWords { static constexpr int n = RB < 4 ? 1 : RB / 4; };

template <int RB>
__device__ __forceinline__ void load_row(const unsigned char *xs, uint32_t row, uint32_t (&r)[RowWords<RB>::n])
{
    const unsigned char *p = xs + (size_t)row * RB;
    if constexpr (RB == 1) r[0] = *p;
    else if constexpr (RB == 2) r[0] = *reinterpret_cast<const uint16_t *>(p);
    else if constexpr (RB == 4) r[0] = *reinterpret_cast<const uint32_t *>(p);
    else if constexpr (RB == 8) { uint2 v = *reinterpret_cast<const uint2 *>(p); r[0] = v.x; r[1] = v.y; }
    else {
#pragma unroll
        for (int i = 0; i < RB / 16; i++) {
            uint4 v = reinterpret_cast<const uint4 *>(p)[i];
            r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
    }
}

template <int DT, int MT>
__device__ __forceinline__ void gather_add(typename ActTraits<DT>::acc (&acc)[MT], const unsigned char *xs, uint32_t row)
{
    constexpr int RB = MT * ActTraits<DT>::size;
    uint32_t r[RowWords<RB>::n];
    load_row<RB>(xs, row, r);
    if constexpr (DT == SPTMM_I8) {
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] += (int32_t)(int8_t)(r[m >> 2] >> (8 * (m & 3)));
    } else if constexpr (DT == SPTMM_F16) {
        if constexpr (MT == 1) {
            acc[0] += __half2float(__ushort_as_half((unsigned short)r[0]));
        } else {
#pragma unroll
            for (int m = 0; m < MT; m += 2) {
                float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&r[m >> 1]));
                acc[m] += f.x; acc[m + 1] += f.y;
            }
        }
    } else {
#pragma unroll
        for (int m = 0; m < MT; m++) acc[m] += __uint_as_float(r[m]);
    }
}

__device__ __forceinline__ int32_t warp_sum(int32_t v) { return __reduce_add_sync(0xffffffffu, v); }
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Fill the transposed tile from X.  mv = valid rows of this tile (the rest read as zero).
// Lanes run along k so that global reads coalesce and shared writes spread over the banks.
template <int DT, int MT>
__device__ __forceinline__ void stage_x(unsigned char *xs, const void *Xv, uint32_t K, uint32_t M,
                                        uint32_t m0, uint32_t mv, bool x_colmajor)
{
    using elem = typename ActTraits<DT>::elem;
    constexpr int ES = ActTraits<DT>::size;
    elem *dst = reinterpret_cast<elem *>(xs);
    const elem *X = reinterpret_cast<const elem *>(Xv);
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    if (MT == 1 && !x_colmajor && ((reinterpret_cast<uintptr_t>(X + (size_t)m0 * K) & 15) == 0)) {
        const uint32_t vec = (K * ES) / 16;
        const uint4 *src = reinterpret_cast<const uint4 *>(X + (size_t)m0 * K);
        for (uint32_t i = tid; i < vec; i += nt) reinterpret_cast<uint4 *>(xs)[i] = __ldg(src + i);
        for (uint32_t k = vec * (16 / ES) + tid; k < K; k += nt) dst[k] = X[(size_t)m0 * K + k];
    } else {
        for (uint32_t m = 0; m < (uint32_t)MT; m++) {
            if (m < mv) {
                for (uint32_t k = tid; k < K; k += nt)
                    dst[(size_t)k * MT + m] = x_colmajor ? X[(size_t)k * M + m0 + m] : X[(size_t)(m0 + m) * K + k];
            } else {
                for (uint32_t k = tid; k < K; k += nt) dst[(size_t)k * MT + m] = elem(0);
            }
        }
    }
    if (tid < (uint32_t)MT) dst[(size_t)K * MT + tid] = elem(0);     // the zero row
}

__host__ __device__ inline size_t xs_bytes(uint32_t K, int rb) { return (((size_t)K + 1) * rb + 15) & ~(size_t)15; }

}  // namespace sptmm
