// Test infrastructure, not product code: C entry points around the REFERENCE's own device kernels, so that the
// GPU tests can run them unmodified on the same inputs as the oracle and the product kernels.
//
// The kernels are not in this repository.  oracle/build_ref.py cuts the kernel-only prefix of the reference's
// single source file (Inference.cu lines 1-292: includes, constants, macros and the kernels dequantAwqKernel,
// rmsNormKernel, applyRotaryKernel, attentionKernel, geluKernel, finalSoftmaxKernel) into a temporary file at
// build time and passes its path as QW3_REF_PREFIX; the rest of the reference does not compile with this
// toolkit.  The launch configurations below are the reference's own (cited per function).
#include QW3_REF_PREFIX

extern "C" {

// dequantAllWeights, Inference.cu:908-1008: one thread per element, 256 threads per block.
int ref_dequant(const void* packed, const void* scale, const void* zp, void* out, int rows, int cols, void* stream) {
    const int TPB = 256, total = rows * cols, grid = (total + TPB - 1) / TPB;
    dequantAwqKernel<<<grid, TPB, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed), static_cast<const half*>(scale), static_cast<const half*>(zp),
        static_cast<half*>(out), rows, cols);
    return (int)cudaGetLastError();
}

// runOneLayer, Inference.cu:1036-1047: one block of 256 threads, 256 floats of shared memory.
int ref_rmsnorm(const void* x, const void* gamma, void* out, int hidden, float eps, void* stream) {
    const int threads = 256;
    rmsNormKernel<<<1, threads, sizeof(float) * threads, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const half*>(x), static_cast<const half*>(gamma), static_cast<half*>(out), hidden, eps);
    return (int)cudaGetLastError();
}

// runOneLayer, Inference.cu:1079-1091: one block per head, one thread per pair; in place.
int ref_rotary(void* q_or_k, const void* cos_table, const void* sin_table, int heads, int head_dim, int pos, void* stream) {
    applyRotaryKernel<<<heads, head_dim / 2, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<half*>(q_or_k), static_cast<const half*>(cos_table), static_cast<const half*>(sin_table), heads,
        head_dim, pos);
    return (int)cudaGetLastError();
}

// runOneLayer, Inference.cu:1192-1197: 256 threads per block; in place.
int ref_gelu(void* x, int len, void* stream) {
    const int TPB = 256;
    geluKernel<<<(len + TPB - 1) / TPB, TPB, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<half*>(x), len);
    return (int)cudaGetLastError();
}

// runOneLayer, Inference.cu:1049-1065 (and 1128, 1176, 1201, 1260): the contraction as the reference calls it, on the
// fp16 buffer dequantAwqKernel wrote: cublasGemmEx(OP_N, OP_N, m = out_dim, n = 1, k = in_dim, A = d_dq with lda = m,
// B = x with ldb = k, C = y with ldc = m), fp16 alpha / beta, tensor-op algorithm.  The compute type the reference
// names, CUBLAS_COMPUTE_16F_FAST_16F, is not an enumerator of this cuBLAS; compute32 == 0 uses CUBLAS_COMPUTE_16F (what
// its fp16 alpha / beta imply), compute32 != 0 CUBLAS_COMPUTE_32F with float alpha / beta (the oracle's arithmetic).
int ref_gemv_cublas(const void* dq, const void* x, void* y, int m, int k, int compute32, void* stream) {
    static cublasHandle_t handle = nullptr;
    if (handle == nullptr && cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) return -1;
    if (cublasSetStream(handle, static_cast<cudaStream_t>(stream)) != CUBLAS_STATUS_SUCCESS) return -2;
    const half alpha_h = __float2half(1.0f), beta_h = __float2half(0.0f);
    const float alpha_f = 1.0f, beta_f = 0.0f;
    const cublasStatus_t st = cublasGemmEx(
        handle, CUBLAS_OP_N, CUBLAS_OP_N, m, 1, k, compute32 ? static_cast<const void*>(&alpha_f) : &alpha_h, dq, CUDA_R_16F, m,
        x, CUDA_R_16F, k, compute32 ? static_cast<const void*>(&beta_f) : &beta_h, y, CUDA_R_16F, m,
        compute32 ? CUBLAS_COMPUTE_32F : CUBLAS_COMPUTE_16F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    return (int)st;
}

}  // extern "C"
