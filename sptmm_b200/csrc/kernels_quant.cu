// kernels_quant.cu -- the activation quantiser as a kernel of its own.
//
// The reference has no quantiser: its activations are int8 from the start (make_X, main.cu:787-797)
// and its results stay int32 (main.cu:591-593).  A layer stack needs the step between two matmuls:
// int32 results -> int8 activations with one scale per row,
//     q = clamp(rint(v * (127 / absmax)), -127, 127),   scale = absmax / 127      (all in fp32).
// The sequence kernel fuses this into its input stage; this is the same arithmetic for callers of
// the per-call entry points (and for the NCCL variant of the layer stack, which quantises what an
// all-gather delivered).  One CTA per row, two passes over the row (it is L2-resident).
#include "device_common.cuh"

namespace sptmm {

struct QuantParams {
    const int32_t *X; int8_t *Xq; float *scale;
    uint32_t M, K, ldx, shard, pair;
};

// element (m, k) of the source: plain rows, or the layout an all-gather of per-rank column shards
// leaves behind -- rank r's M x shard block after rank r-1's
__device__ __forceinline__ int quant_src(const QuantParams &p, uint32_t m, uint32_t k)
{
    if (p.shard == 0) return __ldcg(p.X + (size_t)m * p.ldx + k);
    const uint32_t r = k / p.shard;
    return __ldcg(p.X + ((size_t)r * p.M + m) * p.shard + (k - r * p.shard));
}
__device__ __forceinline__ int quant_value(const QuantParams &p, uint32_t m, uint32_t k)
{
    return p.pair ? quant_src(p, m, 2 * k) + quant_src(p, m, 2 * k + 1) : quant_src(p, m, k);
}

__global__ void __launch_bounds__(512) k_quant_absmax(const QuantParams p)
{
    __shared__ int part[16];
    const uint32_t m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    int amax = 0;
    for (uint32_t k = tid; k < p.K; k += blockDim.x) amax = max(amax, abs(quant_value(p, m, k)));
    amax = __reduce_max_sync(0xffffffffu, amax);
    if (lane == 0) part[warp] = amax;
    __syncthreads();
    amax = 0;
    for (uint32_t w = 0; w < (blockDim.x >> 5); w++) amax = max(amax, part[w]);
    const float s = amax ? 127.0f / (float)amax : 0.0f;
    for (uint32_t k = tid; k < p.K; k += blockDim.x) {
        const int q = max(-127, min(127, __float2int_rn((float)quant_value(p, m, k) * s)));
        p.Xq[(size_t)m * p.K + k] = (int8_t)q;
    }
    if (tid == 0 && p.scale) p.scale[m] = (float)amax / 127.0f;
}

}  // namespace sptmm

using namespace sptmm;

extern "C" int sptmm_quantize_absmax(const int32_t *X, uint32_t M, uint32_t K, uint32_t ldx, uint32_t shard, uint32_t pair,
                                     int8_t *Xq, float *scale, uint32_t flags, void *stream)
{
    if (!X || !Xq) return fail(SPTMM_ERR_INVALID, "quantize_absmax: null pointer");
    if (M == 0 || K == 0) return fail(SPTMM_ERR_INVALID, "quantize_absmax: M=%u K=%u", M, K);
    const uint32_t width = pair ? 2 * K : K;
    if (shard && pair && (shard & 1)) return fail(SPTMM_ERR_INVALID, "quantize_absmax: pair sums need shards of an even number of columns (%u)", shard);
    if (!shard && ldx && ldx < width) return fail(SPTMM_ERR_INVALID, "quantize_absmax: ldx=%u is less than the %u source columns", ldx, width);
    QuantParams prm{X, Xq, scale, M, K, ldx ? ldx : width, shard, pair ? 1u : 0u};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M); cfg.blockDim = dim3(512); cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (flags & SPTMM_LAUNCH_PDL) ? 1 : 0;
    SPTMM_CUDA_TRY(cudaLaunchKernelEx(&cfg, k_quant_absmax, prm));
    return SPTMM_OK;
}
