// Bias add, rotation of queries and keys, and the write of keys and values into
// the paged cache, in one launch.
//
// qkv [T, (nq + 2 nkv) d] holds the stacked projections, either in the run's dtype
// or as float32 partial sums [splits, T, width] of a K-split product, which are
// added here in split order before the bias.  For every token t and
// head: add the bias in float32 (if any), rotate the first `rot` elements of q and
// k heads by angle = position * inv_freq in float32 (precise sincosf), write q to
// q_out [T, nq d], the rotated key and the raw value to the cache page that holds
// the token's position.
//
// Cache layout per layer: [pages, 2 (K, V), nkv, page_size, d].  The page of
// position p of the request in slot s is block_table[s * max_blocks + p / page_size].
#include "common.cuh"

namespace ifx {

template <typename T>
__global__ void rope_append_kernel(const T* __restrict__ qkv, const float* __restrict__ qkv_partial, int num_splits,
                                   size_t split_stride, const float* __restrict__ bias,
                                   const float* __restrict__ inv_freq, int rot, int interleaved,
                                   const int* __restrict__ positions, const int* __restrict__ token_req,
                                   const int* __restrict__ req_slot, const int* __restrict__ block_table,
                                   int max_blocks, int page_size, int num_pages, T* __restrict__ kv_pool,
                                   T* __restrict__ q_out, int nq, int nkv, int d, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int head = blockIdx.y;                      // [0, nq) q, [nq, nq+nkv) k, then v
  const int width = (nq + 2 * nkv) * d;
  const size_t src_off = (size_t)t * width + (size_t)head * d;
  const T* src = qkv ? qkv + src_off : nullptr;
  const float* psrc = qkv_partial ? qkv_partial + src_off : nullptr;
  auto load = [&](int e) -> float {
    if (psrc == nullptr) return to_f32(src[e]);
    float v = 0.0f;
    for (int s = 0; s < num_splits; ++s) v += psrc[(size_t)s * split_stride + e];
    return v;
  };
  const float* b = bias ? bias + (size_t)head * d : nullptr;
  const int pos = positions[t];

  T* dst;
  bool rotate;
  if (head < nq) {
    dst = q_out + (size_t)t * nq * d + (size_t)head * d;
    rotate = true;
  } else {
    if (!write_cache) return;
    const int is_v = head >= nq + nkv;
    const int g = head - nq - (is_v ? nkv : 0);
    const int slot = req_slot[token_req[t]];
    const int page = block_table[(size_t)slot * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) return;      // never write outside the pool
    dst = kv_pool + ((((size_t)page * 2 + is_v) * nkv + g) * page_size + (pos % page_size)) * d;
    rotate = !is_v;
  }

  const int half_rot = rot / 2;
  for (int j = threadIdx.x; j < d / 2; j += blockDim.x) {
    int e0, e1;
    bool turn = rotate && j < half_rot;
    if (j < half_rot) {
      e0 = interleaved ? 2 * j : j;
      e1 = interleaved ? 2 * j + 1 : j + half_rot;
    } else {
      e0 = rot + 2 * (j - half_rot);
      e1 = e0 + 1;
    }
    float a = load(e0), c = load(e1);
    if (b) {
      a += b[e0];
      c += b[e1];
    }
    if (turn) {
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      const float ra = a * cs - c * sn;
      const float rc = a * sn + c * cs;
      a = ra;
      c = rc;
    }
    dst[e0] = from_f32<T>(a);
    dst[e1] = from_f32<T>(c);
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" int ifx_rope_append(const void* qkv, const float* qkv_partial, int num_splits, const float* bias, const float* inv_freq, int rot,
                               int interleaved, const int* positions, const int* token_req,
                               const int* req_slot, const int* block_table, int max_blocks, int page_size,
                               int num_pages, void* kv_pool, void* q_out, int num_tokens, int nq, int nkv,
                               int d, int write_cache, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || d % 2 || rot < 0 || rot > d || rot % 2) return IFX_E_BADARG;
  if (rot > 0 && inv_freq == nullptr) return IFX_E_BADARG;
  if (write_cache && (page_size <= 0 || max_blocks <= 0 || kv_pool == nullptr)) return IFX_E_BADARG;
  if (nq + 2 * nkv > 65535) return IFX_E_TOOBIG;
  if ((qkv == nullptr) == (qkv_partial == nullptr)) return IFX_E_BADARG;
  if (qkv_partial != nullptr && num_splits <= 0) return IFX_E_BADARG;
  const size_t split_stride = (size_t)num_tokens * (nq + 2 * nkv) * d;
  dim3 grid(num_tokens, nq + 2 * nkv);
  int threads = d / 2 >= 64 ? 64 : 32;
  if (dtype == IFX_DT_F32)
    return launch_pdl(rope_append_kernel<float>, grid, dim3(threads), 0, stream, 1, (const float*)qkv, qkv_partial,
                      num_splits, split_stride, bias, inv_freq, rot, interleaved, positions, token_req, req_slot,
                      block_table, max_blocks, page_size, num_pages, (float*)kv_pool, (float*)q_out, nq, nkv, d,
                      write_cache);
  if (dtype == IFX_DT_BF16)
    return launch_pdl(rope_append_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, 1,
                      (const __nv_bfloat16*)qkv, qkv_partial, num_splits, split_stride, bias, inv_freq, rot,
                      interleaved, positions, token_req, req_slot, block_table, max_blocks, page_size, num_pages,
                      (__nv_bfloat16*)kv_pool, (__nv_bfloat16*)q_out, nq, nkv, d, write_cache);
  return IFX_E_DTYPE;
}
