// Made-up weights that do not depend on where they are made: element i of a tensor is
// a function of (seed, tensor name, i) alone.  The same arithmetic is restated with
// numpy integers and single float32 operations in weights/random_init.py, and a test
// holds the two bit-equal.
//
// Two Philox4x32-10 blocks, key (seed low word, seed high word ^ crc32(name)), counter
// (i low, i high, block, 0), give sixteen 16-bit integers.  Their sum is an exact integer;
// centred and scaled it is a variable of variance 1 whose excess kurtosis, -6/(5*16), is
// taken out to first order by z + c (z^3 - 3 z), c = 0.075 / 24.  Every float32 step is one
// correctly rounded operation (no fused multiply-add), so every device and the host agree.
#include "common.cuh"

namespace ifx {

__device__ __forceinline__ void philox4x32_10(uint32_t key0, uint32_t key1, uint32_t c0, uint32_t c1, uint32_t c2,
                                              uint32_t c3, uint32_t out[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ key0, n2 = hi0 ^ c3 ^ key1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    key0 += W0;
    key1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ float counter_normal(uint32_t key0, uint32_t key1, unsigned long long i) {
  int sum = 0;
#pragma unroll
  for (uint32_t block = 0; block < 2; ++block) {
    uint32_t w[4];
    philox4x32_10(key0, key1, (uint32_t)i, (uint32_t)(i >> 32), block, 0u, w);
#pragma unroll
    for (int j = 0; j < 4; ++j) sum += (int)(w[j] & 0xFFFFu) + (int)(w[j] >> 16);
  }
  const float t = (float)(2 * sum - 16 * 65535);                 // exact: |t| < 2^24
  const float z = __fmul_rn(t, 6.6072494e-06f);                  // 1 / (2 sqrt(16 (65536^2 - 1) / 12))
  const float z3 = __fmul_rn(__fmul_rn(z, z), z);
  const float corr = __fmul_rn(0.003125f, __fsub_rn(z3, __fmul_rn(3.0f, z)));
  return __fadd_rn(z, corr);
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, unsigned long long n, uint32_t key0, uint32_t key1,
                                     float mean, float std) {
  unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    const float v = __fadd_rn(mean, __fmul_rn(std, counter_normal(key0, key1, i)));
    if constexpr (sizeof(T) == 4) out[i] = v;
    else out[i] = __float2bfloat16_rn(v);
  }
}

}  // namespace ifx

// out[n] = mean + std * z(seed, name, i) in float32 (dt 0) or rounded once to bfloat16 (dt 1).
extern "C" int ifx_random_normal(void* out, long long n, unsigned key0, unsigned key1, float mean, float std, int dt,
                                 cudaStream_t stream) {
  if (n < 0) return IFX_E_BADARG;
  if (n == 0) return 0;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dt == IFX_DT_F32)
    ifx::random_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (unsigned long long)n, key0, key1, mean, std);
  else if (dt == IFX_DT_BF16)
    ifx::random_normal_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((__nv_bfloat16*)out, (unsigned long long)n,
                                                                             key0, key1, mean, std);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}
