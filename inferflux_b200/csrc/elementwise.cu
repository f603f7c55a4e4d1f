// Row and element kernels: embedding gather, RMSNorm (plain and fused with the
// residual sum), SiLU*up, residual add, row gather, block-table scatter.
// The residual stream is float32; norms reduce in float32.
#include "common.cuh"

namespace ifx {

int g_pdl_enabled = 1;
int g_shared_carveout = 100;

// ------------------------------------------------------------------ embedding
// out[t, :] = table[token[t], :] widened to float32.  A token id outside the
// table (the host refuses those before launch) gives a row of zeros, never a read
// outside the table.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int hidden, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = tokens[t];
  float* o = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const T* row = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
}

// -------------------------------------------------------------------- RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w.  ADD = 1: x += delta first (x is updated in
// place) and the norm is taken of the sum.  ADD = 2: the delta arrives as float32
// partial sums [splits, rows, hidden] of a K-split matrix product; they are added
// in split order, so the result does not depend on timing.  One block per row.
// Four consecutive elements of a row of T as floats, through one load or store.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, int ADD>
__global__ void rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ delta_raw,
                               const float* __restrict__ w, T* __restrict__ out, int hidden, float eps,
                               int num_splits, size_t split_stride) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  float* xr = x + row * hidden;
  const T* dr = ADD == 1 ? reinterpret_cast<const T*>(delta_raw) + row * hidden : nullptr;
  const float* pr = ADD == 2 ? reinterpret_cast<const float*>(delta_raw) + row * hidden : nullptr;
  T* o = out + row * hidden;
  const bool vec = (hidden & 3) == 0;                    // rows start 16-byte aligned then (8-byte for bfloat16)
  constexpr int KEEP = 4;                                // the row's elements stay in registers between the passes
  float4 keep[KEEP];
  float ss = 0.0f;
  auto take = [&](int i) -> float4 {                     // x (+ delta) at columns i .. i + 3, written back
    float4 v = *reinterpret_cast<const float4*>(xr + i);
    if (ADD == 1) {
      const float4 d = load4(dr + i);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      *reinterpret_cast<float4*>(xr + i) = v;
    } else if (ADD == 2) {
      float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < num_splits; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(pr + (size_t)s * split_stride + i);
        d.x += p.x; d.y += p.y; d.z += p.z; d.w += p.w;
      }
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      *reinterpret_cast<float4*>(xr + i) = v;
    }
    return v;
  };
  const int step4 = blockDim.x * 4;
  if (vec) {
#pragma unroll
    for (int c = 0; c < KEEP; ++c) {
      const int i = threadIdx.x * 4 + c * step4;
      keep[c] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < hidden) keep[c] = take(i);
      ss += keep[c].x * keep[c].x + keep[c].y * keep[c].y + keep[c].z * keep[c].z + keep[c].w * keep[c].w;
    }
    for (int i = threadIdx.x * 4 + KEEP * step4; i < hidden; i += step4) {
      const float4 v = take(i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = xr[i];
      if (ADD == 1) {
        v += to_f32(dr[i]);
        xr[i] = v;
      } else if (ADD == 2) {
        float d = 0.0f;
        for (int s = 0; s < num_splits; ++s) d += pr[(size_t)s * split_stride + i];
        v += d;
        xr[i] = v;
      }
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)hidden + eps);
  if (vec) {
    auto put = [&](int i, float4 v) {
      const float4 wv = *reinterpret_cast<const float4*>(w + i);
      store4(o + i, make_float4(v.x * r * wv.x, v.y * r * wv.y, v.z * r * wv.z, v.w * r * wv.w));
    };
#pragma unroll
    for (int c = 0; c < KEEP; ++c) {
      const int i = threadIdx.x * 4 + c * step4;
      if (i < hidden) put(i, keep[c]);
    }
    for (int i = threadIdx.x * 4 + KEEP * step4; i < hidden; i += step4) put(i, *reinterpret_cast<const float4*>(xr + i));
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(xr[i] * r * w[i]);
  }
}

// x += sum of K-split partial sums, then RMSNorm, spread over many blocks: block
// (row, chunk) adds the slices of its 512 columns in split order, updates x and
// leaves its sum of squares in `sumsq[row, chunk]`; the block that finishes a row
// last (a ticket counter per row, reset for the next launch) adds the chunk sums in
// chunk order and writes the normalised row.  Nothing waits on another block.
// Loads are issued in batches before anything depends on them: with a handful of
// rows the kernel's time is a few round trips to L2, not bandwidth.
constexpr int kNormChunk = 512;
constexpr int kNormBatch = 12;

template <typename T>
__global__ void __launch_bounds__(128)
reduce_add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ part, const float* __restrict__ w,
                          T* __restrict__ out, int hidden, float eps, int num_splits, size_t split_stride,
                          float* __restrict__ sumsq, int* __restrict__ tickets, int chunks) {
  __shared__ float scratch[32];
  __shared__ int is_last;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, chunk = blockIdx.y;
  float* xr = x + (size_t)row * hidden;
  const float* pr = part + (size_t)row * hidden;
  const int c0 = chunk * kNormChunk + threadIdx.x * 4;
  float ss = 0.0f;
  if (c0 + 3 < hidden && (hidden & 3) == 0) {
    float4 v = *reinterpret_cast<float4*>(xr + c0);
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < num_splits; s0 += kNormBatch) {
      float4 p[kNormBatch];
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j)
        p[j] = s0 + j < num_splits ? __ldcg(reinterpret_cast<const float4*>(pr + (size_t)(s0 + j) * split_stride + c0))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j) {
        d.x += p[j].x; d.y += p[j].y; d.z += p[j].z; d.w += p[j].w;
      }
    }
    v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    *reinterpret_cast<float4*>(xr + c0) = v;
    ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  } else {
    for (int c = c0; c < min(c0 + 4, hidden); ++c) {
      float d = 0.0f;
      for (int s = 0; s < num_splits; ++s) d += pr[(size_t)s * split_stride + c];
      const float v = xr[c] + d;
      xr[c] = v;
      ss += v * v;
    }
  }
  __threadfence();                       // this thread's part of x is out before the ticket is taken
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) {
    sumsq[(size_t)row * chunks + chunk] = ss;
    __threadfence();
    const int t = atomicAdd(&tickets[row], 1);
    is_last = (t == chunks - 1);
    if (is_last) tickets[row] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float total = 0.0f;
  for (int c = 0; c < chunks; ++c) total += __ldcg(&sumsq[(size_t)row * chunks + c]);
  const float r = rsqrtf(total / (float)hidden + eps);
  T* o = out + (size_t)row * hidden;
  if ((hidden & 3) == 0) {
    const int n4 = hidden >> 2;
    for (int i0 = threadIdx.x; i0 < n4; i0 += 128 * kNormBatch) {
      float4 xv[kNormBatch], wv[kNormBatch];
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j) {
        const int i = i0 + j * 128;
        if (i < n4) {
          xv[j] = __ldcg(reinterpret_cast<const float4*>(xr) + i);
          wv[j] = *(reinterpret_cast<const float4*>(w) + i);
        }
      }
#pragma unroll
      for (int j = 0; j < kNormBatch; ++j) {
        const int i = i0 + j * 128;
        if (i < n4) {
          T* dst = o + (size_t)i * 4;
          dst[0] = from_f32<T>(xv[j].x * r * wv[j].x);
          dst[1] = from_f32<T>(xv[j].y * r * wv[j].y);
          dst[2] = from_f32<T>(xv[j].z * r * wv[j].z);
          dst[3] = from_f32<T>(xv[j].w * r * wv[j].w);
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(__ldcg(&xr[i]) * r * w[i]);
  }
}

// The norm without its row scale: x += delta (K-split partial sums, a tensor, or nothing),
// pre = x * w rounded to T, and sumsq[row, chunk] = the chunk's sum of x^2.  The scale
// rsqrt(sum(sumsq[row, :]) / hidden + eps) is a per-row scalar, so the matrix product that
// consumes `pre` applies it to its accumulator instead (pre . W^T is linear in it): no block
// has to wait for a row's other chunks, and the norm costs one pass over 512 columns a block.
// MODE 0: no delta; 1: delta in T; 2: float32 partial sums [splits, rows, hidden].
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
prenorm_kernel(float* __restrict__ x, const void* __restrict__ delta_raw, const float* __restrict__ w,
               T* __restrict__ pre, int hidden, int num_splits, size_t split_stride, float* __restrict__ sumsq,
               int chunks) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  const int row = blockIdx.x, chunk = blockIdx.y;
  float* xr = x + (size_t)row * hidden;
  T* pr = pre + (size_t)row * hidden;
  const int c0 = chunk * kNormChunk + threadIdx.x * 4;
  const bool wide = c0 + 3 < hidden && (hidden & 3) == 0;
  float4 wv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (wide) wv = *reinterpret_cast<const float4*>(w + c0);         // the norm's weight is nobody's output
  pdl_wait();
  float ss = 0.0f;
  if (wide) {
    float4 v = *reinterpret_cast<const float4*>(xr + c0);
    if (MODE == 1) {
      const T* d = reinterpret_cast<const T*>(delta_raw) + (size_t)row * hidden + c0;
      v.x += to_f32(d[0]); v.y += to_f32(d[1]); v.z += to_f32(d[2]); v.w += to_f32(d[3]);
    } else if (MODE == 2) {
      const float* p = reinterpret_cast<const float*>(delta_raw) + (size_t)row * hidden + c0;
      float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s0 = 0; s0 < num_splits; s0 += kNormBatch) {
        float4 q[kNormBatch];
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j)
          q[j] = s0 + j < num_splits ? __ldcg(reinterpret_cast<const float4*>(p + (size_t)(s0 + j) * split_stride))
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kNormBatch; ++j) {
          d.x += q[j].x; d.y += q[j].y; d.z += q[j].z; d.w += q[j].w;
        }
      }
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    if (MODE != 0) *reinterpret_cast<float4*>(xr + c0) = v;
    pr[c0] = from_f32<T>(v.x * wv.x);
    pr[c0 + 1] = from_f32<T>(v.y * wv.y);
    pr[c0 + 2] = from_f32<T>(v.z * wv.z);
    pr[c0 + 3] = from_f32<T>(v.w * wv.w);
    ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  } else {
    for (int c = c0; c < min(c0 + 4, hidden); ++c) {
      float v = xr[c];
      if (MODE == 1) {
        v += to_f32(reinterpret_cast<const T*>(delta_raw)[(size_t)row * hidden + c]);
      } else if (MODE == 2) {
        const float* p = reinterpret_cast<const float*>(delta_raw) + (size_t)row * hidden + c;
        float d = 0.0f;
        for (int s = 0; s < num_splits; ++s) d += __ldcg(p + (size_t)s * split_stride);
        v += d;
      }
      if (MODE != 0) xr[c] = v;
      pr[c] = from_f32<T>(v * w[c]);
      ss += v * v;
    }
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) sumsq[(size_t)row * chunks + chunk] = ss;
}

// out = pre * rsqrt(sum(sumsq[row, :]) / hidden + eps): the plain tensor of a pre-normed row.
template <typename T>
__global__ void scale_rows_kernel(const T* __restrict__ pre, const float* __restrict__ sumsq, T* __restrict__ out,
                                  int hidden, int chunks, float eps) {
  const int row = blockIdx.x;
  float total = 0.0f;
  for (int c = 0; c < chunks; ++c) total += sumsq[(size_t)row * chunks + c];
  const float r = rsqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[(size_t)row * hidden + i] = from_f32<T>(to_f32(pre[(size_t)row * hidden + i]) * r);
}

// ------------------------------------------------------------------- SiLU*up
// in [rows, 2*inter] = gate | up;  out[r, i] = silu(gate) * up, silu(g) = g / (1 + exp(-g)).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  size_t r = idx / inter;
  int i = (int)(idx - r * inter);
  float g = to_f32(in[r * 2 * inter + i]);
  float u = to_f32(in[r * 2 * inter + inter + i]);
  out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// bf16, inter % 8 == 0: 16-byte loads, two chunks of 8 elements a thread (four loads in flight).
__global__ void __launch_bounds__(256)
silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int inter,
                       size_t total8) {
  const size_t half = (total8 + 1) / 2;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (first >= half) return;
  const int per_row = inter / 8;
  size_t idx[2] = {first, first + half};
  uint4 gv[2], uv[2];
  size_t row[2];
  int col[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (idx[i] >= total8) idx[i] = first;                       // an odd count: the second chunk repeats the first
    row[i] = idx[i] / per_row;
    col[i] = (int)(idx[i] - row[i] * per_row) * 8;
    gv[i] = __ldcs(reinterpret_cast<const uint4*>(in + row[i] * 2 * inter + col[i]));
    uv[i] = __ldcs(reinterpret_cast<const uint4*>(in + row[i] * 2 * inter + inter + col[i]));
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv[i]);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv[i]);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 g = __bfloat1622float2(g2[k]);
      float2 u = __bfloat1622float2(u2[k]);
      // exp and the division through the special-function unit: their error (a few float32 ulps) is far
      // below the rounding of the bfloat16 result, and the kernel stays bound by memory, not by issue slots
      float a = __fdividef(g.x, 1.0f + __expf(-g.x)) * u.x;
      float b = __fdividef(g.y, 1.0f + __expf(-g.y)) * u.y;
      o2[k] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<uint4*>(out + row[i] * inter + col[i]) = ov;
  }
}

template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) x[idx] += to_f32(delta[idx]);
}

// x += sum over splits of float32 partial sums [splits, rows*hidden], in split order.
__global__ void residual_add_partial_kernel(float* __restrict__ x, const float* __restrict__ part, size_t total,
                                            int num_splits) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float d = 0.0f;
  for (int s0 = 0; s0 < num_splits; s0 += 8) {             // eight loads in flight, added in split order
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = s0 + j < num_splits ? __ldcg(&part[(size_t)(s0 + j) * total + idx]) : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) d += v[j];
  }
  x[idx] += d;
}

// out = sum over splits (+ bias[col]) rounded to T: the plain way to consume partial sums.
template <typename T>
__global__ void reduce_partial_kernel(const float* __restrict__ part, const float* __restrict__ bias,
                                      T* __restrict__ out, size_t total, int cols, int num_splits) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float d = 0.0f;
  for (int s = 0; s < num_splits; ++s) d += part[(size_t)s * total + idx];
  if (bias) d += bias[idx % cols];
  out[idx] = from_f32<T>(d);
}

__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int hidden, int num_src_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  int src = rows[r];
  float* o = out + (size_t)r * hidden;
  if (src < 0 || src >= num_src_rows) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    return;
  }
  const float* s = x + (size_t)src * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = s[i];
}

__global__ void scatter_i32_kernel(int* __restrict__ table, const int* __restrict__ index,
                                   const int* __restrict__ value, int n, int table_size) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int at = index[i];
  if (at >= 0 && at < table_size) table[at] = value[i];
}

// dst[dst_index[i]] = src[src_index[i]]: tokens sampled by the previous step go straight into
// this step's token ids without passing through the host.
__global__ void relay_i32_kernel(int* __restrict__ dst, const int* __restrict__ dst_index, const int* __restrict__ src,
                                 const int* __restrict__ src_index, int n, int dst_size, int src_size) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = dst_index[i], s = src_index[i];
  if (d >= 0 && d < dst_size && s >= 0 && s < src_size) dst[d] = src[s];
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// 1 (default): kernels of the decode chain overlap their start with the previous kernel's end.
// Percent of an SM's memory the chain's kernels prefer as shared memory (-1: leave it to the driver).
int ifx_set_shared_carveout(int percent) {
  g_shared_carveout = percent;
  return 0;
}

int ifx_set_pdl(int enabled) {
  g_pdl_enabled = enabled ? 1 : 0;
  return 0;
}

int ifx_embed(const void* table, const int* tokens, float* out, int num_tokens, int hidden, int vocab,
              int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return IFX_E_BADARG;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == IFX_DT_F32)
    return launch_pdl(embed_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, 1, (const float*)table, tokens, out,
                      hidden, vocab);
  else if (dtype == IFX_DT_BF16)
    return launch_pdl(embed_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream, 1,
                      (const __nv_bfloat16*)table, tokens, out, hidden, vocab);
  return IFX_E_DTYPE;
}

// delta == nullptr: plain norm of x.  Otherwise x += delta, then the norm of the sum;
// num_splits > 0 says that delta is float32 partial sums [num_splits, rows, hidden].
int ifx_rmsnorm(float* x, const void* delta, const float* w, void* out, int rows, int hidden, float eps,
                int num_splits, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0 || num_splits < 0) return IFX_E_BADARG;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t stride = (size_t)rows * hidden;
#define IFX_NORM(T, ADD)                                                                                        \
  return launch_pdl(rmsnorm_kernel<T, ADD>, dim3(rows), dim3(threads), 0, stream, 1, x, delta, w, (T*)out, hidden, eps, \
                    num_splits, stride)
  if (dtype == IFX_DT_F32) {
    if (!delta) IFX_NORM(float, 0);
    else if (num_splits > 0) IFX_NORM(float, 2);
    else IFX_NORM(float, 1);
  } else if (dtype == IFX_DT_BF16) {
    if (!delta) IFX_NORM(__nv_bfloat16, 0);
    else if (num_splits > 0) IFX_NORM(__nv_bfloat16, 2);
    else IFX_NORM(__nv_bfloat16, 1);
  }
#undef IFX_NORM
  return IFX_E_DTYPE;
}

// The same as ifx_rmsnorm with partial sums, over many blocks.  sumsq: float32
// [rows, ceil(hidden / 512)] scratch; tickets: int32 [rows], zero before the first call
// (the kernel leaves them zero).
int ifx_reduce_add_rmsnorm(float* x, const float* part, const float* w, void* out, int rows, int hidden, float eps,
                           int num_splits, float* sumsq, int* tickets, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0 || num_splits <= 0 || sumsq == nullptr || tickets == nullptr) return IFX_E_BADARG;
  const int chunks = (hidden + kNormChunk - 1) / kNormChunk;
  if (chunks > 65535) return IFX_E_TOOBIG;
  dim3 grid(rows, chunks);
  const size_t stride = (size_t)rows * hidden;
  if (dtype == IFX_DT_F32)
    return launch_pdl(reduce_add_rmsnorm_kernel<float>, grid, dim3(128), 0, stream, 1, x, part, w, (float*)out, hidden,
                      eps, num_splits, stride, sumsq, tickets, chunks);
  if (dtype == IFX_DT_BF16)
    return launch_pdl(reduce_add_rmsnorm_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, 1, x, part, w,
                      (__nv_bfloat16*)out, hidden, eps, num_splits, stride, sumsq, tickets, chunks);
  return IFX_E_DTYPE;
}

// sumsq: float32 [rows, ceil(hidden / 512)].  delta == nullptr: no add; num_splits > 0: float32 partial sums.
int ifx_prenorm(float* x, const void* delta, const float* w, void* pre, float* sumsq, int rows, int hidden,
                int num_splits, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0 || num_splits < 0 || sumsq == nullptr) return IFX_E_BADARG;
  const int chunks = (hidden + kNormChunk - 1) / kNormChunk;
  if (chunks > 65535) return IFX_E_TOOBIG;
  dim3 grid(rows, chunks);
  const size_t stride = (size_t)rows * hidden;
#define IFX_PRE(T, MODE) \
  return launch_pdl(prenorm_kernel<T, MODE>, grid, dim3(128), 0, stream, 1, x, delta, w, (T*)pre, hidden, num_splits, \
                    stride, sumsq, chunks)
  if (dtype == IFX_DT_F32) {
    if (!delta) IFX_PRE(float, 0);
    if (num_splits > 0) IFX_PRE(float, 2);
    IFX_PRE(float, 1);
  }
  if (dtype == IFX_DT_BF16) {
    if (!delta) IFX_PRE(__nv_bfloat16, 0);
    if (num_splits > 0) IFX_PRE(__nv_bfloat16, 2);
    IFX_PRE(__nv_bfloat16, 1);
  }
#undef IFX_PRE
  return IFX_E_DTYPE;
}

int ifx_scale_rows(const void* pre, const float* sumsq, void* out, int rows, int hidden, float eps, int dtype,
                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int chunks = (hidden + kNormChunk - 1) / kNormChunk;
  if (dtype == IFX_DT_F32)
    scale_rows_kernel<float><<<rows, 256, 0, stream>>>((const float*)pre, sumsq, (float*)out, hidden, chunks, eps);
  else if (dtype == IFX_DT_BF16)
    scale_rows_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>((const __nv_bfloat16*)pre, sumsq, (__nv_bfloat16*)out,
                                                               hidden, chunks, eps);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_residual_add_partial(float* x, const float* part, int rows, int hidden, int num_splits, cudaStream_t stream) {
  if (rows <= 0 || num_splits <= 0) return 0;
  const size_t total = (size_t)rows * hidden;
  return launch_pdl(residual_add_partial_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, 1, x, part,
                    total, num_splits);
}

int ifx_reduce_partial(const float* part, const float* bias, void* out, int rows, int cols, int num_splits, int dtype,
                       cudaStream_t stream) {
  if (rows <= 0 || num_splits <= 0) return 0;
  const size_t total = (size_t)rows * cols;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == IFX_DT_F32)
    reduce_partial_kernel<float><<<blocks, 256, 0, stream>>>(part, bias, (float*)out, total, cols, num_splits);
  else if (dtype == IFX_DT_BF16)
    reduce_partial_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(part, bias, (__nv_bfloat16*)out, total, cols,
                                                                     num_splits);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_silu_mul(const void* gate_up, void* out, int rows, int inter, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter <= 0) return IFX_E_BADARG;
  const size_t total = (size_t)rows * inter;
  if (dtype == IFX_DT_BF16 && inter % 8 == 0 && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const size_t total8 = total / 8;
    silu_mul_bf16x8_kernel<<<(unsigned)(((total8 + 1) / 2 + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total8);
  } else if (dtype == IFX_DT_BF16) {
    silu_mul_kernel<__nv_bfloat16><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
  } else if (dtype == IFX_DT_F32) {
    silu_mul_kernel<float><<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((const float*)gate_up, (float*)out,
                                                                               inter, total);
  } else {
    return IFX_E_DTYPE;
  }
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_residual_add(float* x, const void* delta, int rows, int hidden, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t total = (size_t)rows * hidden;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == IFX_DT_F32)
    residual_add_kernel<float><<<blocks, 256, 0, stream>>>(x, (const float*)delta, total);
  else if (dtype == IFX_DT_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(x, (const __nv_bfloat16*)delta, total);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_gather_rows(const float* x, const int* rows, float* out, int num_rows, int hidden, int num_src_rows,
                    cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  return launch_pdl(gather_rows_kernel, dim3(num_rows), dim3(256), 0, stream, 1, x, rows, out, hidden, num_src_rows);
}

int ifx_relay_i32(int* dst, const int* dst_index, const int* src, const int* src_index, int n, int dst_size,
                  int src_size, cudaStream_t stream) {
  if (n <= 0) return 0;
  relay_i32_kernel<<<(n + 127) / 128, 128, 0, stream>>>(dst, dst_index, src, src_index, n, dst_size, src_size);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_scatter_i32(int* table, const int* index, const int* value, int n, int table_size, cudaStream_t stream) {
  if (n <= 0) return 0;
  scatter_i32_kernel<<<(n + 127) / 128, 128, 0, stream>>>(table, index, value, n, table_size);
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
