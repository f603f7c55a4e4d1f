// Library matrix product for the bfloat16 path: C[M, N] = A[M, K] . W[N, K]^T with
// float32 accumulation, through cublasGemmEx exactly as the reference calls it
// (runtime/backends/cuda/native/cublas_gemm.cpp:98-116: OP_T on the weight with
// lda = K, OP_N on the activations, CUBLAS_COMPUTE_32F).  The output may be
// bfloat16 or float32 (the LM head writes float32 logits directly).
//
// One handle per device, made at first use with a workspace of its own so that
// calls can be captured into CUDA graphs.
#include <cublas_v2.h>

#include "common.cuh"

namespace {

constexpr int kMaxDevices = 16;
constexpr size_t kWorkspaceBytes = 64ull << 20;

struct PerDevice {
  cublasHandle_t handle = nullptr;
  void* workspace = nullptr;
};
PerDevice g_dev[kMaxDevices];

int get_handle(cublasHandle_t* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return IFX_E_TOOBIG;
  PerDevice& pd = g_dev[dev];
  if (!pd.handle) {
    if (cublasCreate(&pd.handle) != CUBLAS_STATUS_SUCCESS) return IFX_E_BADARG;
    e = cudaMalloc(&pd.workspace, kWorkspaceBytes);
    if (e != cudaSuccess) return (int)e;
    if (cublasSetWorkspace(pd.handle, pd.workspace, kWorkspaceBytes) != CUBLAS_STATUS_SUCCESS) return IFX_E_BADARG;
  }
  *out = pd.handle;
  return 0;
}

}  // namespace

// Makes the handle and its workspace.  Call it once before any stream capture.
extern "C" int ifx_cublas_init() {
  cublasHandle_t h;
  return get_handle(&h);
}

// out_dtype: IFX_DT_BF16 or IFX_DT_F32.  A and W are bfloat16.  Returns 1000 + the
// cuBLAS status if the library refuses the call.
extern "C" int ifx_gemm_cublas_bf16(const void* A, const void* W, void* C, int M, int N, int K, int out_dtype,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return IFX_E_BADARG;
  cublasHandle_t h;
  int rc = get_handle(&h);
  if (rc) return rc;
  if (cublasSetStream(h, stream) != CUBLAS_STATUS_SUCCESS) return IFX_E_BADARG;
  const float alpha = 1.0f, beta = 0.0f;
  cudaDataType ctype = out_dtype == IFX_DT_F32 ? CUDA_R_32F : CUDA_R_16BF;
  if (out_dtype != IFX_DT_F32 && out_dtype != IFX_DT_BF16) return IFX_E_DTYPE;
  cublasStatus_t st = cublasGemmEx(h, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, W, CUDA_R_16BF, K, A, CUDA_R_16BF,
                                   K, &beta, C, ctype, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (st != CUBLAS_STATUS_SUCCESS) return 1000 + (int)st;
  return 0;
}
