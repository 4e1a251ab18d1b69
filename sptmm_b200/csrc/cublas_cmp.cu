// cublas_cmp.cu -- dense comparator: int8 x int8 -> int32 through cublasGemmEx with the
// operand layout of the reference's call (main.cu:856-867).  A reported reference only; the
// ternary kernels never call into cuBLAS.
#include <cublas_v2.h>

#include "device_common.cuh"

using namespace sptmm;

static int cublas_handle(cublasHandle_t *out)
{
    static thread_local cublasHandle_t handle = nullptr;
    static thread_local int handle_device = -1;
    int dev = 0;
    SPTMM_CUDA_TRY(cudaGetDevice(&dev));
    if (!handle || handle_device != dev) {
        if (handle) cublasDestroy(handle);
        handle = nullptr;
        cublasStatus_t s = cublasCreate(&handle);
        if (s != CUBLAS_STATUS_SUCCESS) return fail(SPTMM_ERR_CUDA, "cublasCreate failed: %d", (int)s);
        handle_device = dev;
    }
    *out = handle;
    return SPTMM_OK;
}

extern "C" int sptmm_dense_cublas_gemm(const int8_t *X_colmajor, const int8_t *W_dense, int32_t *C_colmajor,
                                       uint32_t M, uint32_t K, uint32_t N, void *stream)
{
    if (!X_colmajor || !W_dense || !C_colmajor)
        return fail(SPTMM_ERR_INVALID, "dense_cublas_gemm: null pointer (the reference passes a null W, main.cu:837)");
    cublasHandle_t handle = nullptr;
    const int hrc = cublas_handle(&handle);
    if (hrc != SPTMM_OK) return hrc;
    cublasSetStream(handle, (cudaStream_t)stream);
    const int alpha = 1, beta = 0;
    cublasStatus_t s = cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_N, (int)M, (int)N, (int)K, &alpha,
                                    X_colmajor, CUDA_R_8I, (int)M, W_dense, CUDA_R_8I, (int)K, &beta,
                                    C_colmajor, CUDA_R_32I, (int)M, CUBLAS_COMPUTE_32I, CUBLAS_GEMM_DEFAULT);
    if (s != CUBLAS_STATUS_SUCCESS)
        return fail(SPTMM_ERR_UNSUPPORTED, "cublasGemmEx(int8, M=%u K=%u N=%u) failed with status %d", M, K, N, (int)s);
    return SPTMM_OK;
}

// The same with fp16 operands and fp32 accumulation and output (the dense comparator of the large
// fp16 sweeps; the reference has no such call).  Column-major as above; W_dense holds -1, 0, +1.
extern "C" int sptmm_dense_cublas_gemm_f16(const void *X_colmajor, const void *W_dense, float *C_colmajor,
                                           uint32_t M, uint32_t K, uint32_t N, void *stream)
{
    if (!X_colmajor || !W_dense || !C_colmajor) return fail(SPTMM_ERR_INVALID, "dense_cublas_gemm_f16: null pointer");
    cublasHandle_t handle = nullptr;
    const int hrc = cublas_handle(&handle);
    if (hrc != SPTMM_OK) return hrc;
    cublasSetStream(handle, (cudaStream_t)stream);
    const float alpha = 1.0f, beta = 0.0f;
    cublasStatus_t s = cublasGemmEx(handle, CUBLAS_OP_N, CUBLAS_OP_N, (int)M, (int)N, (int)K, &alpha,
                                    X_colmajor, CUDA_R_16F, (int)M, W_dense, CUDA_R_16F, (int)K, &beta,
                                    C_colmajor, CUDA_R_32F, (int)M, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (s != CUBLAS_STATUS_SUCCESS)
        return fail(SPTMM_ERR_UNSUPPORTED, "cublasGemmEx(fp16, M=%u K=%u N=%u) failed with status %d", M, K, N, (int)s);
    return SPTMM_OK;
}
