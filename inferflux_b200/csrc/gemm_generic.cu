// C[M, N] = A[M, K] . W[N, K]^T (+ bias[N]) on the CUDA cores, accumulating in
// float32 with one fused multiply-add per product, k ascending.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no reduced
// precision mode) and it takes every M, N and K.  The additions that make one
// output element happen in an order that depends on K alone, so a row's result is
// bit-for-bit the same whatever other rows share the launch.
#include "common.cuh"

namespace ifx {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_nt_kernel(const TI* __restrict__ A, const TI* __restrict__ W,
                                                      const float* __restrict__ bias, TO* __restrict__ C,
                                                      int M, int N, int K) {
  __shared__ float As[BK][BM + PAD];
  __shared__ float Ws[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const bool a_row_ok = (m0 + lr) < M, w_row_ok = (n0 + lr) < N;
  const TI* a_ptr = A + (size_t)(m0 + lr) * K;
  const TI* w_ptr = W + (size_t)(n0 + lr) * K;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_row_ok && k < K) ? to_f32(a_ptr[k]) : 0.0f;
      Ws[lk + i][lr] = (w_row_ok && k < K) ? to_f32(w_ptr[k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      C[(size_t)m * N + n] = from_f32<TO>(v);
    }
  }
}

}  // namespace ifx

using namespace ifx;

// in_dtype: dtype of A and W.  out_dtype: dtype of C (float32 or the input dtype).
extern "C" int ifx_gemm_generic(const void* A, const void* W, const float* bias, void* C, int M, int N, int K,
                                int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return IFX_E_BADARG;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return IFX_E_TOOBIG;
  if (in_dtype == IFX_DT_F32 && out_dtype == IFX_DT_F32)
    gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)A, (const float*)W, bias, (float*)C, M, N, K);
  else if (in_dtype == IFX_DT_BF16 && out_dtype == IFX_DT_BF16)
    gemm_nt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (__nv_bfloat16*)C, M, N, K);
  else if (in_dtype == IFX_DT_BF16 && out_dtype == IFX_DT_F32)
    gemm_nt_kernel<__nv_bfloat16, float><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)W,
                                                                   bias, (float*)C, M, N, K);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}
