// Row and element kernels: embedding gather, RMSNorm (plain and fused with the
// residual sum), SiLU*up, residual add, row gather, block-table scatter.
// The residual stream is float32; norms reduce in float32.
#include "common.cuh"

namespace ifx {

// ------------------------------------------------------------------ embedding
// out[t, :] = table[token[t], :] widened to float32.  A token id outside the
// table (the host refuses those before launch) gives a row of zeros, never a read
// outside the table.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int hidden, int vocab) {
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
// y = x * rsqrt(mean(x^2) + eps) * w.  With ADD, x += delta first (x is updated in
// place) and the norm is taken of the sum.  One block per row.
template <typename T, bool ADD>
__global__ void rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                               const float* __restrict__ w, T* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  float* xr = x + row * hidden;
  const T* dr = ADD ? delta + row * hidden : nullptr;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = xr[i];
    if (ADD) {
      v += to_f32(dr[i]);
      xr[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / (float)hidden + eps);
  T* o = out + row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(xr[i] * r * w[i]);
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

// bf16, inter % 8 == 0: 8 elements per thread through 16-byte loads.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                       int inter, size_t total8) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = inter / 8;
  size_t r = idx / per_row;
  int c = (int)(idx - r * per_row) * 8;
  const uint4 gv = *reinterpret_cast<const uint4*>(in + r * 2 * inter + c);
  const uint4 uv = *reinterpret_cast<const uint4*>(in + r * 2 * inter + inter + c);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 ov;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float2 g = __bfloat1622float2(g2[k]);
    float2 u = __bfloat1622float2(u2[k]);
    float a = g.x / (1.0f + expf(-g.x)) * u.x;
    float b = g.y / (1.0f + expf(-g.y)) * u.y;
    o2[k] = __floats2bfloat162_rn(a, b);
  }
  *reinterpret_cast<uint4*>(out + r * inter + c) = ov;
}

template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ delta, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) x[idx] += to_f32(delta[idx]);
}

__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int hidden, int num_src_rows) {
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

}  // namespace ifx

using namespace ifx;

extern "C" {

int ifx_embed(const void* table, const int* tokens, float* out, int num_tokens, int hidden, int vocab,
              int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden <= 0 || vocab <= 0) return IFX_E_BADARG;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == IFX_DT_F32)
    embed_kernel<float><<<num_tokens, threads, 0, stream>>>((const float*)table, tokens, out, hidden, vocab);
  else if (dtype == IFX_DT_BF16)
    embed_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>((const __nv_bfloat16*)table, tokens, out,
                                                                    hidden, vocab);
  else
    return IFX_E_DTYPE;
  IFX_CHECK_LAUNCH();
  return 0;
}

// delta == nullptr: plain norm of x.  Otherwise x += delta, then the norm of the sum.
int ifx_rmsnorm(float* x, const void* delta, const float* w, void* out, int rows, int hidden, float eps,
                int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0) return IFX_E_BADARG;
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  if (dtype == IFX_DT_F32) {
    if (delta)
      rmsnorm_kernel<float, true><<<rows, threads, 0, stream>>>(x, (const float*)delta, w, (float*)out, hidden, eps);
    else
      rmsnorm_kernel<float, false><<<rows, threads, 0, stream>>>(x, nullptr, w, (float*)out, hidden, eps);
  } else if (dtype == IFX_DT_BF16) {
    if (delta)
      rmsnorm_kernel<__nv_bfloat16, true><<<rows, threads, 0, stream>>>(x, (const __nv_bfloat16*)delta, w,
                                                                        (__nv_bfloat16*)out, hidden, eps);
    else
      rmsnorm_kernel<__nv_bfloat16, false><<<rows, threads, 0, stream>>>(x, nullptr, w, (__nv_bfloat16*)out,
                                                                         hidden, eps);
  } else {
    return IFX_E_DTYPE;
  }
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_silu_mul(const void* gate_up, void* out, int rows, int inter, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (inter <= 0) return IFX_E_BADARG;
  const size_t total = (size_t)rows * inter;
  if (dtype == IFX_DT_BF16 && inter % 8 == 0 && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const size_t total8 = total / 8;
    silu_mul_bf16x8_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, stream>>>(
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
  gather_rows_kernel<<<num_rows, 256, 0, stream>>>(x, rows, out, hidden, num_src_rows);
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
