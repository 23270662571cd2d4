// Library matrix product: out[M, N] (float) = a[M, K] * w[N, K]^T through cuBLAS,
// with float accumulation.  Float inputs run as true 32-bit (CUBLAS_COMPUTE_32F with
// pedantic math: no TF32, no reduced-precision splitting); bfloat16 inputs multiply
// on the tensor cores and accumulate in float.
//
// Parity: runtime/blas.py:41-56 of nehanmohammed19/cuda-inference-serving-runtime binds
// the same library for the same layout ([out, in] weights, C^T = W * X^T).
#include <cublas_v2.h>

#include "common.cuh"

namespace {
cublasHandle_t g_handle = nullptr;
cublasHandle_t g_handle_f32 = nullptr;
}

CISR_EXPORT int cisr_gemm_library_init(void* workspace, long long workspace_bytes) {
    if (!g_handle) {
        if (cublasCreate(&g_handle) != CUBLAS_STATUS_SUCCESS) return -10;
        if (cublasCreate(&g_handle_f32) != CUBLAS_STATUS_SUCCESS) return -10;
        if (cublasSetMathMode(g_handle_f32, CUBLAS_PEDANTIC_MATH) != CUBLAS_STATUS_SUCCESS) return -11;
    }
    if (workspace) {
        // A caller-owned workspace keeps the library from allocating inside a stream capture.
        if (cublasSetWorkspace(g_handle, workspace, (size_t)workspace_bytes / 2) != CUBLAS_STATUS_SUCCESS) return -12;
        if (cublasSetWorkspace(g_handle_f32, (char*)workspace + workspace_bytes / 2, (size_t)workspace_bytes / 2) != CUBLAS_STATUS_SUCCESS) return -12;
    }
    return 0;
}

CISR_EXPORT int cisr_gemm_library(const void* a, const void* w, int dtype, float* out, int m, int n, int k,
                                  void* stream) {
    if (m <= 0 || n <= 0) return 0;
    if (!g_handle) return -13;
    cublasHandle_t h = dtype == CISR_BF16 ? g_handle : g_handle_f32;
    if (cublasSetStream(h, (cudaStream_t)stream) != CUBLAS_STATUS_SUCCESS) return -14;
    const float alpha = 1.f, beta = 0.f;
    const cudaDataType_t t = dtype == CISR_BF16 ? CUDA_R_16BF : CUDA_R_32F;
    cublasStatus_t st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, n, m, k, &alpha, w, t, k, a, t, k, &beta, out,
                                     CUDA_R_32F, n, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    return st == CUBLAS_STATUS_SUCCESS ? 0 : -100 - (int)st;
}
