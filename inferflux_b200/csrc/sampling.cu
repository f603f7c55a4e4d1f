// Sampling from float32 logits [rows, vocab].
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
// Thresholds are found on the bit pattern of the probability (for non-negative floats
// the bit pattern orders like the value) without a sort.  sample_kernel has one block per
// row and bisects (31 passes: the exact k-th largest value, the exact nucleus boundary); the
// sampler the engine uses spreads a row over many blocks and descends by radix (see
// "sampling over many blocks" below): 33 us instead of 142 for a plain temperature draw from
// 152,064 logits, 100 us instead of 1,400 with top-k, min-p and top-p together.
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
  const int bd = blockDim.x;
  int i = threadIdx.x;
  for (; i + 7 * bd < n; i += 8 * bd) {              // eight loads in flight, compared in index order
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = row[i + j * bd] * mul;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v[j] > best.v) best = ArgBest{v[j], i + j * bd};   // strict: the lowest index of a thread's stride wins
  }
  for (; i < n; i += bd) {
    const float v = row[i] * mul;
    if (v > best.v) best = ArgBest{v, i};
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
  pdl_launch_dependents();
  pdl_wait();
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


// ------------------------------------------------------- sampling over many blocks
// The same draw as sample_kernel, but a row is spread over `chunks` blocks and the
// thresholds are found by a radix descent (three levels of 10 bits of the element's
// bit pattern, a histogram of counts and masses per level) instead of 31 passes of
// bisection.  An element is e = exp(logit / T - max), so the largest is exactly 1.  Masses
// are sums of e in fixed point (2^-40), i.e. integers: their sums do not depend on the
// order of the additions, so blocks may add them with atomics and the draw stays
// reproducible.  Passes are separate launches; the block that finishes a row last (a
// ticket per row) does the row's small sequential step and leaves tickets and histograms
// zero for the next use.
constexpr int kBins = 1024;
constexpr int kSmpThreads = 256;
constexpr int kSmpMaxChunks = 32;

struct SampleRowState {
  float inv_t;                    // 1 / temperature
  float rowmax;                   // max of logit / T
  int argidx;                     // where it is (lowest index)
  int flags;                      // bit 0: draws (temperature > 0), 1: top-k, 2: top-p
  unsigned thr_key;               // elements with bits >= thr_key are kept
  unsigned prefix;                // radix descent: the bits fixed so far
  unsigned k_res;                 // top-k descent: how many more elements from the current range
  int pick_chunk;                 // the chunk the draw falls into
  unsigned long long need;        // top-p descent: how much more mass from the current range
  unsigned long long target;      // the draw, as mass inside pick_chunk
  float top_p;
  int pad;
};

__device__ __forceinline__ float smp_elem(const float* __restrict__ row, int i, float inv_t, float rowmax) {
  return expf(row[i] * inv_t - rowmax);
}
__device__ __forceinline__ unsigned long long smp_mass(float e) { return __float2ull_rz(e * 1099511627776.0f); }

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch /* 32 */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned long long r = lane < nwarps ? scratch[lane] : 0ull;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

// Takes the row's ticket; true in every thread of the block that came last.  The caller's writes
// before the call are visible to that block after it.
__device__ __forceinline__ bool smp_last_block(int* tickets, int row, int chunks, int* flag_smem) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&tickets[row], 1);
    *flag_smem = t == chunks - 1;
    if (*flag_smem) tickets[row] = 0;
  }
  __syncthreads();
  const bool last = *flag_smem != 0;
  if (last) __threadfence();
  return last;
}

// From the top bin down: the largest bin b whose suffix (bins >= b) reaches `want`, and the
// suffix above it.  Counts (by_mass = false) or masses.  One block, 256 threads, 4 bins each.
__device__ void smp_scan_bins(const unsigned* __restrict__ cnt, const unsigned long long* __restrict__ mass,
                              bool by_mass, unsigned long long want, int* bin_out, unsigned long long* above_out,
                              unsigned long long* scan_smem /* 256 + 32 */, int* found_smem) {
  const int t = threadIdx.x;                          // thread t owns bins 1023 - 4t ... 1020 - 4t, top first
  unsigned long long v[4], mine = 0ull;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int b = kBins - 1 - (4 * t + j);
    v[j] = by_mass ? __ldcg(&mass[b]) : (unsigned long long)__ldcg(&cnt[b]);
    mine += v[j];
  }
  // inclusive scan over the threads (Hillis-Steele in shared memory; integers: any order gives the same)
  scan_smem[t] = mine;
  if (t == 0) *found_smem = 0x7fffffff;
  __syncthreads();
  for (int off = 1; off < kSmpThreads; off <<= 1) {
    const unsigned long long add = t >= off ? scan_smem[t - off] : 0ull;
    __syncthreads();
    scan_smem[t] += add;
    __syncthreads();
  }
  const unsigned long long incl = scan_smem[t], excl = incl - mine;
  if (excl < want && incl >= want) atomicMin(found_smem, t);
  __syncthreads();
  if (t == *found_smem) {
    unsigned long long run = excl;
    int b = kBins - 1 - 4 * t;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (run + v[j] >= want) {
        b = kBins - 1 - (4 * t + j);
        break;
      }
      run += v[j];
    }
    *bin_out = b;
    *above_out = run;
  }
  if (*found_smem == 0x7fffffff && t == 0) {          // `want` beyond everything there is: the lowest bin
    *bin_out = 0;
    *above_out = 0ull;
  }
  __syncthreads();
}

struct SampleScratch {
  SampleRowState* state;
  int* tickets;
  float* part_val;
  int* part_idx;
  unsigned long long* chunk_mass;
  unsigned* cnt_a;
  unsigned long long* mass_a;
  unsigned* cnt_b;
  unsigned long long* mass_b;
};

__global__ void __launch_bounds__(kSmpThreads)
smp_max_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
               const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
               int* __restrict__ out, int vocab, int chunks, int features, SampleScratch sc) {
  __shared__ ArgBest scratch[32];
  __shared__ int last_flag;
  const int r = blockIdx.x, c = blockIdx.y;
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = min(vocab, c * per), end = min(vocab, begin + per);
  const float temp = temperature[r];
  const bool draws = temp > 0.0f;
  const float inv_t = draws ? 1.0f / temp : 1.0f;
  ArgBest b = block_argmax(logits + (size_t)r * vocab + begin, end - begin, inv_t, scratch);
  if (threadIdx.x == 0) {
    sc.part_val[r * chunks + c] = end > begin ? b.v : -INFINITY;
    sc.part_idx[r * chunks + c] = begin + b.i;
  }
  if (!smp_last_block(sc.tickets, r, chunks, &last_flag) || threadIdx.x >= 32) return;
  ArgBest best{-INFINITY, 0x7fffffff};
  for (int k = threadIdx.x; k < chunks; k += 32) {
    ArgBest o{__ldcg(&sc.part_val[r * chunks + k]), __ldcg(&sc.part_idx[r * chunks + k])};
    best = better(best, o);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) {
    if (best.i == 0x7fffffff) best = ArgBest{0.0f, 0};
    SampleRowState st = {};
    st.inv_t = inv_t;
    st.rowmax = best.v;
    st.argidx = best.i;
    const int k = top_k[r];
    const float tp = top_p[r], mp = min_p[r];
    // a filter whose passes the caller did not ask for (features) is off for the row as well
    st.flags = (draws ? 1 : 0) | ((draws && (features & 1) && k > 0 && k < vocab) ? 2 : 0) |
               ((draws && (features & 2) && tp > 0.0f && tp < 1.0f) ? 4 : 0);
    st.thr_key = (draws && mp > 0.0f) ? __float_as_uint(fminf(mp, 1.0f)) : 0u;   // e >= min_p * (largest e = 1)
    st.k_res = (st.flags & 2) ? (unsigned)k : 0u;
    st.top_p = tp;
    sc.state[r] = st;
    if (!draws) out[r] = best.i;
  }
}

// LEVEL 1, 2, 3: bits [29:20], [19:10], [9:0] of the element.  PURPOSE 0: top-k (counts), 1: top-p (masses).
// Level 1 serves both and lands in histogram A; the others in B.
template <int LEVEL, int PURPOSE>
__global__ void __launch_bounds__(kSmpThreads)
smp_hist_kernel(const float* __restrict__ logits, int vocab, int chunks, SampleScratch sc) {
  __shared__ unsigned cnt_s[kBins];
  __shared__ unsigned long long mass_s[kBins];
  __shared__ unsigned long long scan_s[kSmpThreads + 32];
  __shared__ int last_flag, found_s, bin_s;
  __shared__ unsigned long long above_s;
  const int r = blockIdx.x, c = blockIdx.y;
  const SampleRowState st = sc.state[r];
  const int want_flag = LEVEL == 1 ? 6 : (PURPOSE == 0 ? 2 : 4);
  if (!(st.flags & 1) || !(st.flags & want_flag)) return;
  constexpr int SHIFT = LEVEL == 1 ? 20 : (LEVEL == 2 ? 10 : 0);
  for (int i = threadIdx.x; i < kBins; i += blockDim.x) {
    cnt_s[i] = 0u;
    mass_s[i] = 0ull;
  }
  __syncthreads();
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = min(vocab, c * per), end = min(vocab, begin + per);
  const float* row = logits + (size_t)r * vocab;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float e = smp_elem(row, i, st.inv_t, st.rowmax);
    const unsigned bits = __float_as_uint(e);
    if (LEVEL == 1 || (bits >> (SHIFT + 10)) == st.prefix) {
      const int bin = (bits >> SHIFT) & (kBins - 1);
      atomicAdd(&cnt_s[bin], 1u);
      atomicAdd(&mass_s[bin], smp_mass(e));
    }
  }
  __syncthreads();
  unsigned* cnt_g = (LEVEL == 1 ? sc.cnt_a : sc.cnt_b) + (size_t)r * kBins;
  unsigned long long* mass_g = (LEVEL == 1 ? sc.mass_a : sc.mass_b) + (size_t)r * kBins;
  for (int i = threadIdx.x; i < kBins; i += blockDim.x) {
    if (cnt_s[i]) {
      atomicAdd(&cnt_g[i], cnt_s[i]);
      atomicAdd(&mass_g[i], mass_s[i]);
    }
  }
  if (!smp_last_block(sc.tickets, r, chunks, &last_flag)) return;
  // ---- the row's step: where does the target fall among the bins
  const bool scan_k = LEVEL == 1 ? (st.flags & 2) != 0 : PURPOSE == 0;
  const bool scan_p = LEVEL != 1 && PURPOSE == 1;
  if (scan_k || scan_p) {
    smp_scan_bins(cnt_g, mass_g, scan_p, scan_p ? st.need : (unsigned long long)st.k_res, &bin_s, &above_s, scan_s,
                  &found_s);
    if (threadIdx.x == 0) {
      SampleRowState* g = sc.state + r;
      const unsigned prefix = LEVEL == 1 ? (unsigned)bin_s : ((st.prefix << 10) | (unsigned)bin_s);
      g->prefix = prefix;
      if (scan_p) g->need = st.need - above_s; else g->k_res = st.k_res - (unsigned)above_s;
      if (LEVEL == 3) g->thr_key = max(st.thr_key, prefix);        // the descent has all 30 bits
    }
  }
  // Histogram B is used once per level; A stays for the top-p descent unless the row has none.
  if (LEVEL != 1 || !(st.flags & 4)) {
    __syncthreads();
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) {
      cnt_g[i] = 0u;
      mass_g[i] = 0ull;
    }
  }
}

// Kept mass per chunk.  PASS 0: before the nucleus (rows with top-p start its descent from histogram A
// here; the others get their draw); PASS 1: rows with top-p, after it.
template <int PASS>
__global__ void __launch_bounds__(kSmpThreads)
smp_mass_kernel(const float* __restrict__ logits, const unsigned* __restrict__ seed_lo,
                const unsigned* __restrict__ seed_hi, const unsigned* __restrict__ step, int vocab, int chunks,
                SampleScratch sc) {
  __shared__ unsigned long long scan_s[kSmpThreads + 32];
  __shared__ int last_flag, found_s, bin_s;
  __shared__ unsigned long long above_s;
  const int r = blockIdx.x, c = blockIdx.y;
  const SampleRowState st = sc.state[r];
  if (!(st.flags & 1) || (PASS == 1 && !(st.flags & 4))) return;
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = min(vocab, c * per), end = min(vocab, begin + per);
  const float* row = logits + (size_t)r * vocab;
  unsigned long long mine = 0ull;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float e = smp_elem(row, i, st.inv_t, st.rowmax);
    if (__float_as_uint(e) >= st.thr_key) mine += smp_mass(e);
  }
  const unsigned long long total = block_sum_u64(mine, scan_s);
  if (threadIdx.x == 0) sc.chunk_mass[r * chunks + c] = total;
  if (!smp_last_block(sc.tickets, r, chunks, &last_flag)) return;
  unsigned long long kept = 0ull;
  for (int k = 0; k < chunks; ++k) kept += __ldcg(&sc.chunk_mass[r * chunks + k]);
  if (PASS == 0 && (st.flags & 4)) {
    // nucleus: the smallest set of the largest kept elements whose mass reaches top_p of the kept mass
    unsigned long long need = (unsigned long long)((double)st.top_p * (double)kept);
    if (need < 1ull) need = 1ull;
    if (need > kept) need = kept;
    unsigned* cnt_g = sc.cnt_a + (size_t)r * kBins;
    unsigned long long* mass_g = sc.mass_a + (size_t)r * kBins;
    smp_scan_bins(cnt_g, mass_g, true, need, &bin_s, &above_s, scan_s, &found_s);
    if (threadIdx.x == 0) {
      sc.state[r].prefix = (unsigned)bin_s;
      sc.state[r].need = need - above_s;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins; i += blockDim.x) {
      cnt_g[i] = 0u;
      mass_g[i] = 0ull;
    }
    return;
  }
  if (threadIdx.x == 0) {
    const uint32_t bits = philox_uniform_bits(seed_lo[r], seed_hi[r], step[r], 0u, 0u, 0u);
    const double u = (double)(bits >> 8) * (1.0 / 16777216.0);
    unsigned long long target = (unsigned long long)(u * (double)kept);
    if (kept > 0ull && target >= kept) target = kept - 1ull;
    int pick = -1;
    unsigned long long run = 0ull;
    for (int k = 0; k < chunks; ++k) {
      const unsigned long long m = __ldcg(&sc.chunk_mass[r * chunks + k]);
      if (m > 0ull && target < run + m) {
        pick = k;
        break;
      }
      run += m;
    }
    sc.state[r].pick_chunk = pick;
    sc.state[r].target = target - run;
  }
}

// The draw: in the chosen chunk, the first kept element (in index order) whose running mass exceeds the target.
__global__ void __launch_bounds__(kSmpThreads)
smp_pick_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab, int chunks, SampleScratch sc) {
  __shared__ unsigned long long scan_s[kSmpThreads];
  __shared__ int chosen;
  const int r = blockIdx.x, c = blockIdx.y;
  const SampleRowState st = sc.state[r];
  if (!(st.flags & 1)) return;
  if (st.pick_chunk < 0) {                               // nothing kept (cannot happen: the largest element always is)
    if (c == 0 && threadIdx.x == 0) out[r] = st.argidx;
    return;
  }
  if (c != st.pick_chunk) return;
  const int per = (vocab + chunks - 1) / chunks;
  const int begin = min(vocab, c * per), end = min(vocab, begin + per);
  const int seg = (end - begin + kSmpThreads - 1) / kSmpThreads;
  const int lo = min(end, begin + (int)threadIdx.x * seg), hi = min(end, lo + seg);
  const float* row = logits + (size_t)r * vocab;
  unsigned long long mine = 0ull;
  for (int i = lo; i < hi; ++i) {
    const float e = smp_elem(row, i, st.inv_t, st.rowmax);
    if (__float_as_uint(e) >= st.thr_key) mine += smp_mass(e);
  }
  scan_s[threadIdx.x] = mine;
  if (threadIdx.x == 0) chosen = 0x7fffffff;
  __syncthreads();
  for (int off = 1; off < kSmpThreads; off <<= 1) {
    const unsigned long long add = (int)threadIdx.x >= off ? scan_s[threadIdx.x - off] : 0ull;
    __syncthreads();
    scan_s[threadIdx.x] += add;
    __syncthreads();
  }
  const unsigned long long incl = scan_s[threadIdx.x], excl = incl - mine;
  if (mine > 0ull && excl <= st.target && st.target < incl) atomicMin(&chosen, (int)threadIdx.x);
  __syncthreads();
  if (chosen == 0x7fffffff) {
    if (threadIdx.x == 0) out[r] = st.argidx;
    return;
  }
  if ((int)threadIdx.x != chosen) return;
  unsigned long long run = excl;
  int pick = st.argidx;
  for (int i = lo; i < hi; ++i) {
    const float e = smp_elem(row, i, st.inv_t, st.rowmax);
    if (__float_as_uint(e) >= st.thr_key) {
      run += smp_mass(e);
      if (run > st.target) {
        pick = i;
        break;
      }
    }
  }
  out[r] = pick;
}

static size_t smp_align(size_t v) { return (v + 255) & ~(size_t)255; }

static size_t smp_layout(SampleScratch* sc, unsigned char* base, int rows) {
  size_t off = 0;
  auto take = [&](size_t bytes) {
    unsigned char* p = base ? base + off : nullptr;
    off += smp_align(bytes);
    return p;
  };
  SampleScratch s;
  s.state = reinterpret_cast<SampleRowState*>(take((size_t)rows * sizeof(SampleRowState)));
  s.tickets = reinterpret_cast<int*>(take((size_t)rows * 4));
  s.part_val = reinterpret_cast<float*>(take((size_t)rows * kSmpMaxChunks * 4));
  s.part_idx = reinterpret_cast<int*>(take((size_t)rows * kSmpMaxChunks * 4));
  s.chunk_mass = reinterpret_cast<unsigned long long*>(take((size_t)rows * kSmpMaxChunks * 8));
  s.cnt_a = reinterpret_cast<unsigned*>(take((size_t)rows * kBins * 4));
  s.mass_a = reinterpret_cast<unsigned long long*>(take((size_t)rows * kBins * 8));
  s.cnt_b = reinterpret_cast<unsigned*>(take((size_t)rows * kBins * 4));
  s.mass_b = reinterpret_cast<unsigned long long*>(take((size_t)rows * kBins * 8));
  if (sc) *sc = s;
  return off;
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
  return launch_pdl(argmax_chunks_kernel, dim3(rows, chunks), dim3(256), 0, stream, 1, logits, out, vocab, chunks,
                    part_val, part_idx, tickets);
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

// Bytes of scratch ifx_sample_blocks needs for up to `capacity` rows.  The scratch must be zero before
// its first use; the kernels leave it ready for the next call with the same capacity (the places of its
// parts depend on the capacity, not on a call's rows).
long long ifx_sample_scratch_bytes(int capacity) {
  return (long long)smp_layout(nullptr, nullptr, capacity < 1 ? 1 : capacity);
}

// The draw of ifx_sample with every row spread over many blocks.  features: bit 0 = some row has top-k,
// bit 1 = some row has top-p (the passes those need are launched only then; a row without them skips them).
int ifx_sample_blocks(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                      const float* min_p, const unsigned* seed_lo, const unsigned* seed_hi, const unsigned* step,
                      int* out, int rows, int vocab, int features, void* scratch, int capacity,
                      cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || rows > 65535 || scratch == nullptr) return IFX_E_BADARG;
  if (rows > capacity) return IFX_E_TOOBIG;
  SampleScratch sc;
  smp_layout(&sc, static_cast<unsigned char*>(scratch), capacity);
  int chunks = vocab / 2048;
  chunks = chunks < 1 ? 1 : (chunks > kSmpMaxChunks ? kSmpMaxChunks : chunks);
  const dim3 grid(rows, chunks);
  smp_max_kernel<<<grid, kSmpThreads, 0, stream>>>(logits, temperature, top_k, top_p, min_p, out, vocab, chunks, features,
                                                    sc);
  if (features & 3) smp_hist_kernel<1, 0><<<grid, kSmpThreads, 0, stream>>>(logits, vocab, chunks, sc);
  if (features & 1) {
    smp_hist_kernel<2, 0><<<grid, kSmpThreads, 0, stream>>>(logits, vocab, chunks, sc);
    smp_hist_kernel<3, 0><<<grid, kSmpThreads, 0, stream>>>(logits, vocab, chunks, sc);
  }
  smp_mass_kernel<0><<<grid, kSmpThreads, 0, stream>>>(logits, seed_lo, seed_hi, step, vocab, chunks, sc);
  if (features & 2) {
    smp_hist_kernel<2, 1><<<grid, kSmpThreads, 0, stream>>>(logits, vocab, chunks, sc);
    smp_hist_kernel<3, 1><<<grid, kSmpThreads, 0, stream>>>(logits, vocab, chunks, sc);
    smp_mass_kernel<1><<<grid, kSmpThreads, 0, stream>>>(logits, seed_lo, seed_hi, step, vocab, chunks, sc);
  }
  smp_pick_kernel<<<grid, kSmpThreads, 0, stream>>>(logits, out, vocab, chunks, sc);
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
