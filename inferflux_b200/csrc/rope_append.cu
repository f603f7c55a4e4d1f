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
                                   T* __restrict__ q_out, int nq, int nkv, int d, int write_cache,
                                   int early_dependents) {
  // The attention kernel behind this one is let in early only if the caller says so: a grid of it that fills
  // the SMs would sit on shared memory and fetch keys against the weights of the q/k/v product still running in
  // front (a decode step of the 7B shape at batch 8: 3.07 ms without, 3.24 ms with); a small one gains its
  // prologue (batch 1: 358 against 350 tokens/s).
  if (early_dependents) pdl_launch_dependents();
  // Positions, slots, the block table, the bias and the angles do not come from the kernel in front:
  // they are fetched and the sines computed before it is known to have finished.
  const int t = blockIdx.x;
  const int head = blockIdx.y;                      // [0, nq) q, [nq, nq+nkv) k, then v
  const int width = (nq + 2 * nkv) * d;
  const size_t src_off = (size_t)t * width + (size_t)head * d;
  const T* src = qkv ? qkv + src_off : nullptr;
  const float* psrc = qkv_partial ? qkv_partial + src_off : nullptr;
  auto load2 = [&](int e0, int e1, float& a, float& c) {     // the two elements of a pair, K slices added in order
    if (psrc == nullptr) {
      a = to_f32(src[e0]);
      c = to_f32(src[e1]);
      return;
    }
    a = c = 0.0f;
    for (int s0 = 0; s0 < num_splits; s0 += 8) {                // 16 loads in flight a round
      float va[8], vc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = s0 + j < num_splits;
        va[j] = in ? __ldcg(psrc + (size_t)(s0 + j) * split_stride + e0) : 0.0f;
        vc[j] = in ? __ldcg(psrc + (size_t)(s0 + j) * split_stride + e1) : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a += va[j];
        c += vc[j];
      }
    }
  };
  const float* b = bias ? bias + (size_t)head * d : nullptr;
  const int pos = positions[t];

  T* dst = nullptr;
  bool rotate = true;
  if (head < nq) {
    dst = q_out + (size_t)t * nq * d + (size_t)head * d;
  } else if (write_cache) {
    const int is_v = head >= nq + nkv;
    const int g = head - nq - (is_v ? nkv : 0);
    const int slot = req_slot[token_req[t]];
    const int page = block_table[(size_t)slot * max_blocks + pos / page_size];
    if (page >= 0 && page < num_pages)              // never write outside the pool
      dst = kv_pool + ((((size_t)page * 2 + is_v) * nkv + g) * page_size + (pos % page_size)) * d;
    rotate = !is_v;
  }

  const int half_rot = rot / 2;
  struct Pair {
    int e0, e1;
    bool turn;
    float sn, cs, b0, b1;
  };
  auto prepare = [&](int j) -> Pair {
    Pair p;
    p.turn = rotate && j < half_rot;
    if (j < half_rot) {
      p.e0 = interleaved ? 2 * j : j;
      p.e1 = interleaved ? 2 * j + 1 : j + half_rot;
    } else {
      p.e0 = rot + 2 * (j - half_rot);
      p.e1 = p.e0 + 1;
    }
    p.b0 = b ? b[p.e0] : 0.0f;
    p.b1 = b ? b[p.e1] : 0.0f;
    p.sn = 0.0f;
    p.cs = 1.0f;
    if (p.turn) sincosf((float)pos * inv_freq[j], &p.sn, &p.cs);
    return p;
  };
  Pair first = {};
  if ((int)threadIdx.x < d / 2) first = prepare(threadIdx.x);
  pdl_wait();
  if (dst == nullptr) return;
  for (int j = threadIdx.x; j < d / 2; j += blockDim.x) {
    const Pair p = j == (int)threadIdx.x ? first : prepare(j);
    float a, c;
    load2(p.e0, p.e1, a, c);
    a += p.b0;
    c += p.b1;
    if (p.turn) {
      const float ra = a * p.cs - c * p.sn;
      const float rc = a * p.sn + c * p.cs;
      a = ra;
      c = rc;
    }
    if (head >= nq) {                 // the cache only ever holds finite values: a masked key's value gets the
      a = isfinite(a) ? a : 0.0f;     // weight zero, and zero times it must be zero whoever wrote it
      c = isfinite(c) ? c : 0.0f;
    }
    dst[p.e0] = from_f32<T>(a);
    dst[p.e1] = from_f32<T>(c);
  }
}

// The same work for many tokens (prompt portions): one block per token.  The cosines
// and sines of a token's angles are the same for all its heads, so they are computed
// once into shared memory; then every thread moves 8 + 8 elements (a 16-byte chunk and
// its rotation partner half a head away) per step.  Takes the common case only:
// bfloat16 activations (not partial sums), whole-head split-half rotation, head
// sizes that are multiples of 16.
__global__ void __launch_bounds__(1024)
rope_append_rows_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ bias,
                        const float* __restrict__ inv_freq, const int* __restrict__ positions,
                        const int* __restrict__ token_req, const int* __restrict__ req_slot,
                        const int* __restrict__ block_table, int max_blocks, int page_size, int num_pages,
                        __nv_bfloat16* __restrict__ kv_pool, __nv_bfloat16* __restrict__ q_out, int nq, int nkv, int d,
                        int write_cache) {
  __shared__ float cs[128], sn[128];                    // d / 2 <= 128
  const int t = blockIdx.x;
  const int half = d / 2;
  const int width = (nq + 2 * nkv) * d;
  const int cph = half / 8;                             // 16-byte chunks per half head
  const int items = (nq + 2 * nkv) * cph;
  const __nv_bfloat16* row = qkv + (size_t)t * width;
  // The block has one thread per item where it can; the item's loads go out before the chain
  // position -> angles and token -> slot -> page is followed.
  int it = threadIdx.x;
  uint4 lo_raw = make_uint4(0u, 0u, 0u, 0u), hi_raw = lo_raw;
  if (it < items) {
    const int head = it / cph, c = (it % cph) * 8;
    lo_raw = *reinterpret_cast<const uint4*>(row + head * d + c);
    hi_raw = *reinterpret_cast<const uint4*>(row + head * d + half + c);
  }
  const int pos = positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sn[j], &cs[j]);
  size_t page_base = 0;
  bool page_ok = false;
  if (write_cache) {
    const int slot = req_slot[token_req[t]];
    const int page = block_table[(size_t)slot * max_blocks + pos / page_size];
    page_ok = page >= 0 && page < num_pages;
    page_base = (size_t)page * 2 * nkv * page_size * d + (size_t)(pos % page_size) * d;
  }
  __syncthreads();
  for (; it < items; it += blockDim.x) {
    const int head = it / cph, c = (it % cph) * 8;
    if (it != (int)threadIdx.x) {                        // more items than threads: the later ones load here
      lo_raw = *reinterpret_cast<const uint4*>(row + head * d + c);
      hi_raw = *reinterpret_cast<const uint4*>(row + head * d + half + c);
    }
    const bool is_q = head < nq, is_v = head >= nq + nkv;
    __nv_bfloat16* dst;
    if (is_q) {
      dst = q_out + (size_t)t * nq * d + (size_t)head * d;
    } else {
      if (!write_cache || !page_ok) continue;
      const int g = head - nq - (is_v ? nkv : 0);
      dst = kv_pool + page_base + ((size_t)(is_v ? nkv : 0) + g) * page_size * d;
    }
    float blo[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, bhi[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (bias) {                                          // d % 16 == 0: both runs of 8 floats are 32-byte aligned
      const float4* bl = reinterpret_cast<const float4*>(bias + head * d + c);
      const float4* bh = reinterpret_cast<const float4*>(bias + head * d + half + c);
      *reinterpret_cast<float4*>(blo) = bl[0];
      *reinterpret_cast<float4*>(blo + 4) = bl[1];
      *reinterpret_cast<float4*>(bhi) = bh[0];
      *reinterpret_cast<float4*>(bhi + 4) = bh[1];
    }
    const __nv_bfloat162* lo2 = reinterpret_cast<const __nv_bfloat162*>(&lo_raw);
    const __nv_bfloat162* hi2 = reinterpret_cast<const __nv_bfloat162*>(&hi_raw);
    uint4 lo_out, hi_out;
    __nv_bfloat162* lo_o = reinterpret_cast<__nv_bfloat162*>(&lo_out);
    __nv_bfloat162* hi_o = reinterpret_cast<__nv_bfloat162*>(&hi_out);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = __bfloat1622float2(lo2[k]), b = __bfloat1622float2(hi2[k]);
      a.x += blo[2 * k];
      a.y += blo[2 * k + 1];
      b.x += bhi[2 * k];
      b.y += bhi[2 * k + 1];
      if (!is_v) {
        const float c0 = cs[c + 2 * k], s0 = sn[c + 2 * k], c1 = cs[c + 2 * k + 1], s1 = sn[c + 2 * k + 1];
        const float ax = a.x * c0 - b.x * s0, bx = a.x * s0 + b.x * c0;
        const float ay = a.y * c1 - b.y * s1, by = a.y * s1 + b.y * c1;
        a = make_float2(ax, ay);
        b = make_float2(bx, by);
      }
      if (!is_q) {                    // the cache only ever holds finite values
        a.x = isfinite(a.x) ? a.x : 0.0f;
        a.y = isfinite(a.y) ? a.y : 0.0f;
        b.x = isfinite(b.x) ? b.x : 0.0f;
        b.y = isfinite(b.y) ? b.y : 0.0f;
      }
      lo_o[k] = __floats2bfloat162_rn(a.x, a.y);
      hi_o[k] = __floats2bfloat162_rn(b.x, b.y);
    }
    *reinterpret_cast<uint4*>(dst + c) = lo_out;
    *reinterpret_cast<uint4*>(dst + half + c) = hi_out;
  }
}

}  // namespace ifx

using namespace ifx;

extern "C" int ifx_rope_append(const void* qkv, const float* qkv_partial, int num_splits, const float* bias, const float* inv_freq, int rot,
                               int interleaved, const int* positions, const int* token_req,
                               const int* req_slot, const int* block_table, int max_blocks, int page_size,
                               int num_pages, void* kv_pool, void* q_out, int num_tokens, int nq, int nkv,
                               int d, int write_cache, int early_dependents, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || d <= 0 || d % 2 || rot < 0 || rot > d || rot % 2) return IFX_E_BADARG;
  if (rot > 0 && inv_freq == nullptr) return IFX_E_BADARG;
  if (write_cache && (page_size <= 0 || max_blocks <= 0 || kv_pool == nullptr)) return IFX_E_BADARG;
  if (nq + 2 * nkv > 65535) return IFX_E_TOOBIG;
  if ((qkv == nullptr) == (qkv_partial == nullptr)) return IFX_E_BADARG;
  if (qkv_partial != nullptr && num_splits <= 0) return IFX_E_BADARG;
  const size_t split_stride = (size_t)num_tokens * (nq + 2 * nkv) * d;
  if (dtype == IFX_DT_BF16 && qkv != nullptr && num_tokens >= 64 && rot == d && !interleaved && d % 16 == 0 &&
      d <= 256 && (reinterpret_cast<uintptr_t>(qkv) % 16 == 0) && (reinterpret_cast<uintptr_t>(q_out) % 16 == 0) &&
      (kv_pool == nullptr || reinterpret_cast<uintptr_t>(kv_pool) % 16 == 0) &&
      (bias == nullptr || reinterpret_cast<uintptr_t>(bias) % 16 == 0)) {
    const int items = (nq + 2 * nkv) * (d / 16);
    const int threads = items >= 1024 ? 1024 : (items + 31) / 32 * 32;
    rope_append_rows_kernel<<<num_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)qkv, bias, inv_freq, positions, token_req, req_slot, block_table, max_blocks, page_size,
        num_pages, (__nv_bfloat16*)kv_pool, (__nv_bfloat16*)q_out, nq, nkv, d, write_cache);
    IFX_CHECK_LAUNCH();
    return 0;
  }
  dim3 grid(num_tokens, nq + 2 * nkv);
  int threads = d / 2 >= 64 ? 64 : 32;
  if (dtype == IFX_DT_F32)
    return launch_pdl(rope_append_kernel<float>, grid, dim3(threads), 0, stream, 1, (const float*)qkv, qkv_partial,
                      num_splits, split_stride, bias, inv_freq, rot, interleaved, positions, token_req, req_slot,
                      block_table, max_blocks, page_size, num_pages, (float*)kv_pool, (float*)q_out, nq, nkv, d,
                      write_cache, early_dependents);
  if (dtype == IFX_DT_BF16)
    return launch_pdl(rope_append_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, 1,
                      (const __nv_bfloat16*)qkv, qkv_partial, num_splits, split_stride, bias, inv_freq, rot,
                      interleaved, positions, token_req, req_slot, block_table, max_blocks, page_size, num_pages,
                      (__nv_bfloat16*)kv_pool, (__nv_bfloat16*)q_out, nq, nkv, d, write_cache, early_dependents);
  return IFX_E_DTYPE;
}
