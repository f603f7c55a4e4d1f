// Paged causal attention, one warp per (token, query head): the kernel of the
// float32 path and the fallback of the bfloat16 path for sizes the tiled kernels
// do not take.
//
// Every token attends the keys of its own request at positions
// [max(0, pos - window + 1), pos] (window <= 0: from 0), read from the cache
// through the block table; the step's own keys are already in the cache.  Keys
// are visited in chunks of 32 in increasing position; scores, the running
// maximum, the running sum and the output accumulate in float32.  The order of
// every addition depends only on the token's position and the window, so the
// result at a position is bit-for-bit the same however the tokens were cut into
// steps or batched.
//
// `rows`, if given, lists the flat token indices to work on (num_tokens of them);
// otherwise all tokens 0 .. num_tokens - 1 are done.
//
// Head sizes: multiples of 8 up to 256.
#include "common.cuh"

namespace ifx {

constexpr int kMaxHeadDim = 256;
constexpr int kWarpsPerBlock = 4;

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int d) {
  float s = 0.0f;
  for (int e = 0; e < d; e += 4) {
    const float4 kv = *reinterpret_cast<const float4*>(k + e);
    s = fmaf(q[e], kv.x, s);
    s = fmaf(q[e + 1], kv.y, s);
    s = fmaf(q[e + 2], kv.z, s);
    s = fmaf(q[e + 3], kv.w, s);
  }
  return s;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int d) {
  float s = 0.0f;
  for (int e = 0; e < d; e += 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(k + e);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(p[i]);
      s = fmaf(q[e + 2 * i], f.x, s);
      s = fmaf(q[e + 2 * i + 1], f.y, s);
    }
  }
  return s;
}

template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ kv_pool,
                                         const int* __restrict__ block_table, const int* __restrict__ positions,
                                         const int* __restrict__ token_req, const int* __restrict__ req_slot,
                                         const int* __restrict__ rows, T* __restrict__ out, int num_tokens, int nq,
                                         int nkv, int d,
                                         int page_size, int max_blocks, int num_pages, int window, float scale) {
  __shared__ __align__(16) float q_s[kWarpsPerBlock][kMaxHeadDim];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarpsPerBlock + warp;
  if (item >= (long long)num_tokens * nq) return;
  const int t = rows ? rows[item / nq] : (int)(item / nq), h = (int)(item % nq);
  const int g = h / (nq / nkv);
  const int pos = positions[t];
  const int slot = req_slot[token_req[t]];
  const int* table = block_table + (size_t)slot * max_blocks;
  const size_t page_stride = (size_t)2 * nkv * page_size * d;       // elements per page (K and V)
  const size_t head_off_k = (size_t)g * page_size * d;
  const size_t head_off_v = ((size_t)nkv + g) * page_size * d;

  const T* qrow = q + ((size_t)t * nq + h) * d;
  for (int e = lane; e < d; e += 32) q_s[warp][e] = to_f32(qrow[e]);
  __syncwarp();

  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int end = pos + 1;
  float m = -INFINITY, l = 0.0f;
  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;

  for (int base = first; base < end; base += 32) {
    const int j = base + lane;
    const bool valid = j < end;
    float s = -INFINITY;
    size_t row_off = 0;                                  // element offset of key row j inside its page's K part
    int page = 0;
    if (valid) {
      page = table[j / page_size];
      if (page < 0 || page >= num_pages) page = 0;       // a broken table must not read outside the pool
      row_off = (size_t)(j % page_size) * d;
      s = dot_row<T>(q_s[warp], kv_pool + (size_t)page * page_stride + head_off_k + row_off, d) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.0f;
    const float corr = expf(m - m_new);                  // m = -inf at the start: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= corr;
    const int count = min(32, end - base);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int pg = __shfl_sync(0xffffffffu, page, jj);
      const unsigned long long ro = __shfl_sync(0xffffffffu, (unsigned long long)row_off, jj);
      const T* vrow = kv_pool + (size_t)pg * page_stride + head_off_v + (size_t)ro;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < d) acc[i] = fmaf(pj, to_f32(vrow[e]), acc[i]);
      }
    }
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  T* orow = out + ((size_t)t * nq + h) * d;
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < d) orow[e] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" int ifx_attention_generic(const void* q, const void* kv_pool, const int* block_table,
                                     const int* positions, const int* token_req, const int* req_slot,
                                     const int* rows, void* out, int num_tokens, int nq, int nkv, int d, int page_size,
                                     int max_blocks, int num_pages, int window, float scale, int dtype,
                                     cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || d <= 0 || d % 8 || d > kMaxHeadDim || page_size <= 0 || max_blocks <= 0)
    return IFX_E_BADARG;
  const long long items = (long long)num_tokens * nq;
  const unsigned blocks = (unsigned)((items + kWarpsPerBlock - 1) / kWarpsPerBlock);
  if (dtype == IFX_DT_F32)
    attention_generic_kernel<float><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        (const float*)q, (const float*)kv_pool, block_table, positions, token_req, req_slot, rows, (float*)out,
        num_tokens, nq, nkv, d, page_size, max_blocks, num_pages, window, scale);
  else if (dtype == IFX_DT_BF16)
    attention_generic_kernel<__nv_bfloat16><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)kv_pool, block_table, positions, token_req, req_slot,
        rows, (__nv_bfloat16*)out, num_tokens, nq, nkv, d, page_size, max_blocks, num_pages, window, scale);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}
