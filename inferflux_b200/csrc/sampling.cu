// Sampling from float32 logits [rows, vocab], one block per row.
//
// What the reference samples with (runtime/backends/cuda/native/gpu_sampler.cu):
// argmax with ties to the lowest index (:124-156), softmax(logits / temperature)
// (:216-267), a nucleus mask (:273-330), one uniform number and a walk of the
// cumulative distribution in index order that returns the first index whose
// cumulative mass exceeds it (:374-401), and repetition / frequency / presence
// penalties on recently sampled tokens (:22-48).  Here every row has its own
// parameters and its own counter-based random number (Philox4x32-10 keyed by the
// request's seed, counter = the request's step), so a row's draw does not depend
// on what else is in the batch.  top-k and min-p thresholds are taken as well.
//
// Thresholds are found by bisection on the bit pattern of the probability (for
// non-negative floats the bit pattern orders like the value), which gives the
// exact k-th largest value, or the exact nucleus boundary, in 31 passes without a sort.
#include "common.cuh"

namespace ifx {

constexpr int kSampleThreads = 1024;

struct ArgBest {
  float v;
  int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgBest block_argmax(const float* __restrict__ row, int n, float mul, ArgBest* scratch /* 32 */) {
  ArgBest best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = row[i] * mul;
    if (v > best.v) best = ArgBest{v, i};            // strict: the lowest index of a thread's stride wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  ArgBest r = lane < nwarps ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
    r = better(r, other);
  }
  if (r.i == 0x7fffffff) r.i = 0;                    // a row of NaN or -inf only
  return r;
}

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
  __shared__ ArgBest scratch[32];
  const float* row = logits + (size_t)blockIdx.x * vocab;
  ArgBest b = block_argmax(row, vocab, 1.0f, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = b.i;
}

// Argmax of long rows over many blocks: block (row, chunk) finds the best of its
// slice, the block that finishes a row last (a ticket per row, reset for the next
// launch) picks among the chunk results, the lower index winning ties.
__global__ void argmax_chunks_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, int chunks,
                                     float* __restrict__ part_val, int* __restrict__ part_idx,
                                     int* __restrict__ tickets) {
  __shared__ ArgBest scratch[32];
  __shared__ int is_last;
  const int row = blockIdx.x, chunk = blockIdx.y;
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = min(vocab, chunk * per), end = min(vocab, begin + per);
  const float* base = logits + (size_t)row * vocab;
  ArgBest b = block_argmax(base + begin, end - begin, 1.0f, scratch);
  if (threadIdx.x == 0) {
    part_val[row * chunks + chunk] = end > begin ? b.v : -INFINITY;
    part_idx[row * chunks + chunk] = begin + b.i;
    __threadfence();
    const int t = atomicAdd(&tickets[row], 1);
    is_last = t == chunks - 1;
    if (is_last) tickets[row] = 0;
  }
  __syncthreads();
  if (!is_last || threadIdx.x >= 32) return;
  __threadfence();
  ArgBest best{-INFINITY, 0x7fffffff};
  for (int c = threadIdx.x; c < chunks; c += 32) {
    ArgBest o{__ldcg(&part_val[row * chunks + c]), __ldcg(&part_idx[row * chunks + c])};
    best = better(best, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) out[row] = best.i == 0x7fffffff ? 0 : best.i;
}

// ------------------------------------------------------------------ penalties
// For each distinct recent token of a row (tokens[r, i], counts[r, i] > 0):
// logit = logit > 0 ? logit / rep : logit * rep;  logit -= freq * count;  logit -= pres.
__global__ void penalties_kernel(float* __restrict__ logits, const int* __restrict__ tokens,
                                 const int* __restrict__ counts, const float* __restrict__ rep,
                                 const float* __restrict__ freq, const float* __restrict__ pres, int width,
                                 int vocab) {
  const int r = blockIdx.x;
  float* row = logits + (size_t)r * vocab;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int tok = tokens[(size_t)r * width + i];
    const int cnt = counts[(size_t)r * width + i];
    if (tok < 0 || tok >= vocab || cnt <= 0) continue;
    float v = row[tok];
    v = v > 0.0f ? v / rep[r] : v * rep[r];
    v -= freq[r] * (float)cnt;
    v -= pres[r];
    row[tok] = v;
  }
}

__global__ void logit_bias_kernel(float* __restrict__ logits, const int* __restrict__ rows,
                                  const int* __restrict__ tokens, const float* __restrict__ bias, int n,
                                  int num_rows, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = rows[i], t = tokens[i];
  if (r < 0 || r >= num_rows || t < 0 || t >= vocab) return;
  atomicAdd(&logits[(size_t)r * vocab + t], bias[i]);
}

// --------------------------------------------------------------------- Philox
__device__ __forceinline__ uint32_t philox_uniform_bits(uint32_t key0, uint32_t key1, uint32_t c0, uint32_t c1,
                                                        uint32_t c2, uint32_t c3) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ key0, n1 = lo1, n2 = hi0 ^ c3 ^ key1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    key0 += W0;
    key1 += W1;
  }
  return c0;
}

__device__ __forceinline__ float count_or_mass(const float* __restrict__ p, int n, float thr, float floor_thr,
                                               bool mass, float* scratch) {
  float acc = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = p[i];
    if (v >= thr && v >= floor_thr) acc += mass ? v : 1.0f;
  }
  return block_sum(acc, scratch);
}

// probs: scratch [rows, vocab].  Per row: temperature (<= 0: argmax), top_k (<= 0
// or >= vocab: off), top_p (>= 1: off), min_p (<= 0: off), seed (two words), step.
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, float* __restrict__ probs, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const unsigned* __restrict__ seed_lo, const unsigned* __restrict__ seed_hi,
              const unsigned* __restrict__ step, int* __restrict__ out, int vocab) {
  __shared__ ArgBest abest[32];
  __shared__ float scratch[32];
  __shared__ float seg_incl[kSampleThreads];
  __shared__ int chosen_thread, last_kept, result;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * vocab;
  float* p = probs + (size_t)r * vocab;
  const float temp = temperature[r];

  if (!(temp > 0.0f)) {
    ArgBest b = block_argmax(row, vocab, 1.0f, abest);
    if (threadIdx.x == 0) out[r] = b.i;
    return;
  }
  const float inv_t = 1.0f / temp;
  const ArgBest top = block_argmax(row, vocab, inv_t, abest);
  float part = 0.0f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float e = expf(row[i] * inv_t - top.v);
    p[i] = e;
    part += e;
  }
  const float total = block_sum(part, scratch);
  const float inv_total = 1.0f / total;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) p[i] *= inv_total;
  __syncthreads();
  const float p_max = inv_total;                       // exp(0) / total

  // ---- thresholds: keep p >= thr
  float thr = 0.0f;
  const int k = top_k[r];
  if (k > 0 && k < vocab) {
    unsigned lo = 0u, hi = __float_as_uint(p_max);
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      const float c = count_or_mass(p, vocab, __uint_as_float(mid), 0.0f, false, scratch);
      if (c >= (float)k) lo = mid; else hi = mid - 1u;
    }
    thr = __uint_as_float(lo);
  }
  const float mp = min_p[r];
  if (mp > 0.0f) thr = fmaxf(thr, mp * p_max);
  const float tp = top_p[r];
  if (tp > 0.0f && tp < 1.0f) {
    const float kept = count_or_mass(p, vocab, thr, 0.0f, true, scratch);
    const float need = tp * kept;
    unsigned lo = __float_as_uint(thr), hi = __float_as_uint(p_max);
    while (lo < hi) {
      const unsigned mid = lo + (hi - lo + 1u) / 2u;
      const float m = count_or_mass(p, vocab, __uint_as_float(mid), thr, true, scratch);
      if (m >= need) lo = mid; else hi = mid - 1u;
    }
    thr = __uint_as_float(lo);
  }

  // ---- walk the kept mass in index order
  const int seg = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, (int)threadIdx.x * seg), end = min(vocab, begin + seg);
  float mine = 0.0f;
  int my_last = -1;
  for (int i = begin; i < end; ++i) {
    const float v = p[i];
    if (v >= thr) {
      mine += v;
      my_last = i;
    }
  }
  if (threadIdx.x == 0) {
    chosen_thread = 0x7fffffff;
    last_kept = -1;
    result = -1;
  }
  seg_incl[threadIdx.x] = mine;
  __syncthreads();
  // inclusive scan over the segments (Hillis-Steele; the order of additions is fixed)
  for (int off = 1; off < (int)blockDim.x; off <<= 1) {
    float add = threadIdx.x >= (unsigned)off ? seg_incl[threadIdx.x - off] : 0.0f;
    __syncthreads();
    seg_incl[threadIdx.x] += add;
    __syncthreads();
  }
  const float kept_total = seg_incl[blockDim.x - 1];
  const uint32_t bits = philox_uniform_bits(seed_lo[r], seed_hi[r], step[r], 0u, 0u, 0u);
  const float u = (float)(bits >> 8) * (1.0f / 16777216.0f);
  const float target = u * kept_total;
  const float incl = seg_incl[threadIdx.x], excl = incl - mine;
  if (my_last >= 0) atomicMax(&last_kept, my_last);
  if (mine > 0.0f && incl > target) atomicMin(&chosen_thread, (int)threadIdx.x);
  __syncthreads();
  if ((int)threadIdx.x == chosen_thread) {
    float run = excl;
    int pick = my_last;
    for (int i = begin; i < end; ++i) {
      const float v = p[i];
      if (v >= thr) {
        run += v;
        if (run > target) {
          pick = i;
          break;
        }
      }
    }
    result = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = result >= 0 ? result : (last_kept >= 0 ? last_kept : top.i);
}

}  // namespace ifx

using namespace ifx;

extern "C" {

int ifx_argmax(const float* logits, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return IFX_E_BADARG;
  argmax_kernel<<<rows, 1024, 0, stream>>>(logits, out, vocab);
  IFX_CHECK_LAUNCH();
  return 0;
}

// scratch: part_val float32 [rows, chunks], part_idx int32 [rows, chunks], tickets int32 [rows]
// (zero before the first call; the kernel leaves them zero).
int ifx_argmax_chunks(const float* logits, int* out, int rows, int vocab, int chunks, float* part_val, int* part_idx,
                      int* tickets, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || chunks <= 0 || chunks > 1024) return IFX_E_BADARG;
  dim3 grid(rows, chunks);
  argmax_chunks_kernel<<<grid, 256, 0, stream>>>(logits, out, vocab, chunks, part_val, part_idx, tickets);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_penalties(float* logits, const int* tokens, const int* counts, const float* rep, const float* freq,
                  const float* pres, int rows, int width, int vocab, cudaStream_t stream) {
  if (rows <= 0 || width <= 0) return 0;
  penalties_kernel<<<rows, 64, 0, stream>>>(logits, tokens, counts, rep, freq, pres, width, vocab);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_logit_bias(float* logits, const int* rows_idx, const int* tokens, const float* bias, int n, int rows,
                   int vocab, cudaStream_t stream) {
  if (n <= 0) return 0;
  logit_bias_kernel<<<(n + 127) / 128, 128, 0, stream>>>(logits, rows_idx, tokens, bias, n, rows, vocab);
  IFX_CHECK_LAUNCH();
  return 0;
}

int ifx_sample(const float* logits, float* probs, const float* temperature, const int* top_k, const float* top_p,
               const float* min_p, const unsigned* seed_lo, const unsigned* seed_hi, const unsigned* step, int* out,
               int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return IFX_E_BADARG;
  sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, probs, temperature, top_k, top_p, min_p, seed_lo, seed_hi,
                                                     step, out, vocab);
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // extern "C"

// --------------------------------------------------------------- no allocation
// See no_alloc.h.  The scratch of the many-block argmax as a fixed array in the
// library image, for callers that cannot allocate: [rows x chunks] best values, then
// [rows x chunks] best indices, then one ticket per row (padded to 8 bytes a row).
#include "no_alloc.h"

static __device__ __align__(256) unsigned char g_no_alloc_scratch[IFX_NO_ALLOC_SCRATCH_BYTES];

namespace {
constexpr int kNoAllocMaxDevices = 64;
// Device address of g_no_alloc_scratch per device; in host code the array's name is only a
// handle for cudaGetSymbolAddress, never a pointer a kernel may be given.
void* g_no_alloc_ptr[kNoAllocMaxDevices] = {};
}  // namespace

extern "C" int ifx_argmax_no_alloc(const float* logits, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (logits == nullptr || out == nullptr || rows < 0 || vocab <= 0 || vocab > (1 << 30)) return IFX_E_BADARG;
  if (rows > IFX_NO_ALLOC_MAX_ROWS) return IFX_E_TOOBIG;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoAllocMaxDevices) return IFX_E_TOOBIG;
  if (g_no_alloc_ptr[dev] == nullptr) {                 // first call on this device: look the address up
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return IFX_E_BADARG;
    g_no_alloc_ptr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_no_alloc_ptr[dev]);
  float* part_val = reinterpret_cast<float*>(base);
  int* part_idx = reinterpret_cast<int*>(base + (size_t)IFX_NO_ALLOC_MAX_ROWS * IFX_NO_ALLOC_CHUNKS * 4);
  int* tickets = reinterpret_cast<int*>(base + (size_t)IFX_NO_ALLOC_MAX_ROWS * IFX_NO_ALLOC_CHUNKS * 8);
  // the tickets must start at zero whatever an earlier (perhaps failed) call left behind
  e = cudaMemsetAsync(tickets, 0, (size_t)rows * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(rows, IFX_NO_ALLOC_CHUNKS);
  ifx::argmax_chunks_kernel<<<grid, 256, 0, stream>>>(logits, out, vocab, IFX_NO_ALLOC_CHUNKS, part_val, part_idx,
                                                      tickets);
  IFX_CHECK_LAUNCH();
  return 0;
}
