// Weight-streaming matrix product for few tokens on the 5th-generation tensor
// cores: out[M, N] = act[M, K] . W[N, K]^T for M <= 256 (decode batches, short prompts
// and small prompt portions), where the time is the time to read W once.
//
// The operands are swapped: the weight tile is the MMA's A operand (128 weight rows
// = the 128 TMEM lanes) and the M token rows, padded to 16/32/64/128/256, are its N.
// One thread block owns a tile of 128 weight rows and one slice of K:
//
//   warp 0     producer: TMA (cp.async.bulk.tensor, 128-byte swizzle) of the weight
//              tile [128 x 64] and the activation tile [Mpad x 64] per k-block into
//              a ring of shared-memory stages, each guarded by a full/empty mbarrier;
//   warp 1     allocates TMEM and issues tcgen05.mma (kind::f16, bf16 in, fp32
//              accumulators in TMEM); tcgen05.commit frees a stage when its MMAs are done;
//   warps 2-5  epilogue: tcgen05.ld of the accumulator (lane = weight row, column =
//              token), then one of
//                STORE    out[m, n] = acc (+ bias[n]) as bfloat16 or float32,
//                PARTIAL  part[split, m, n] = acc in float32, for consumers that add
//                         the K slices themselves (residual + norm, bias + rotation),
//                SWIGLU   two accumulators (gate rows and up rows of the same
//                         outputs): out[m, n] = silu(gate) * up,
//                SWIGLU64 the same for a narrow product: 64 gate rows and 64 up rows share
//                         one accumulator (lanes 0-63 and 64-127), so that twice as many
//                         blocks stream the weights; the up half crosses to the gate half's
//                         warps through shared memory.
//
// Splitting K gives narrow products (N = 3584) enough blocks to pull the full HBM
// rate; the partial sums stay in L2 until the consumer reads them, in a fixed
// order, so the result does not depend on timing.
//
// No TMA multicast is used.  Every wait on an mbarrier is bounded: a wait that
// runs out sets *error_flag and the block winds down (drains its copies, frees its
// TMEM) instead of spinning.
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ifx {

constexpr int kTileN = 128;       // weight rows per block (MMA M)
constexpr int kTileK = 64;        // bf16 elements per k-block = one 128-byte swizzle row

enum { MODE_STORE = 0, MODE_PARTIAL = 1, MODE_SWIGLU = 2, MODE_SWIGLU64 = 3 };

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
  // K-major tile of 128-byte rows, 128-byte swizzle: 8-row groups 1024 bytes apart.
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
__device__ __forceinline__ void mma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// grid: (ceil(N / 128), splits).  Dynamic shared memory: see skinny_smem_bytes().
template <int NPAD, int MODE>
__global__ void __launch_bounds__(192)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   const float* __restrict__ bias, void* __restrict__ out, float* __restrict__ partials, int M, int N,
                   int K, int kblocks_per_split, int up_row_offset, int out_is_f32, int stages,
                   const float* __restrict__ row_sumsq, int sumsq_chunks, float eps, int* __restrict__ error_flag) {
  constexpr int W_TILES = MODE == MODE_SWIGLU ? 2 : 1;
  constexpr uint32_t W_BYTES = kTileN * kTileK * 2;                 // 16 KB
  constexpr uint32_t A_BYTES = NPAD * kTileK * 2;
  constexpr uint32_t STAGE_BYTES = W_TILES * W_BYTES + A_BYTES;
  constexpr uint32_t TMEM_COLS = (W_TILES * NPAD) < 32 ? 32 : (W_TILES * NPAD);
  extern __shared__ unsigned char smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * STAGE_BYTES);   // full[stages], empty[stages], done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * stages + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * (MODE == MODE_SWIGLU64 ? kTileN / 2 : kTileN);
  const int split = blockIdx.y;
  const int total_kblocks = (K + kTileK - 1) / kTileK;
  const int kb0 = split * kblocks_per_split;
  const int kb1 = min(total_kblocks, kb0 + kblocks_per_split);
  const int num_kb = max(0, kb1 - kb0);

  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + stages), done_bar = smem_addr(bars + 2 * stages);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(done_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      // The weights do not depend on the kernel before this one: the first ring of weight tiles is
      // on its way before the activations are known to be ready.
      const uint64_t stream_once = l2_evict_first_policy();
      const int early = min(stages, num_kb);
      for (int i = 0; i < early; ++i) {
        const uint32_t dst = smem_addr(smem + (size_t)i * STAGE_BYTES);
        const uint32_t bar = full0 + 8 * i;
        mbar_expect_tx(bar, STAGE_BYTES);
        const int kx = (kb0 + i) * kTileK;
        tma_load_2d_hint(dst, &map_w, kx, n0, bar, stream_once);
        if (MODE == MODE_SWIGLU) tma_load_2d_hint(dst + W_BYTES, &map_w, kx, up_row_offset + n0, bar, stream_once);
        if (MODE == MODE_SWIGLU64) tma_load_2d_hint(dst + W_BYTES / 2, &map_w, kx, up_row_offset + n0, bar, stream_once);
      }
      pdl_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(smem_addr(smem + (size_t)i * STAGE_BYTES) + W_TILES * W_BYTES, &map_a, (kb0 + i) * kTileK, 0,
                    full0 + 8 * i);
      issued = early;
      for (int i = early; i < num_kb && ok; ++i) {
        const int s = i % stages;
        ok = mbar_wait(empty0 + 8 * s, ((i / stages) & 1) ^ 1);
        if (!ok) break;
        const uint32_t dst = smem_addr(smem + (size_t)s * STAGE_BYTES);
        const uint32_t bar = full0 + 8 * s;
        mbar_expect_tx(bar, STAGE_BYTES);
        const int kx = (kb0 + i) * kTileK;
        tma_load_2d_hint(dst, &map_w, kx, n0, bar, stream_once);
        if (MODE == MODE_SWIGLU) tma_load_2d_hint(dst + W_BYTES, &map_w, kx, up_row_offset + n0, bar, stream_once);
        if (MODE == MODE_SWIGLU64) tma_load_2d_hint(dst + W_BYTES / 2, &map_w, kx, up_row_offset + n0, bar, stream_once);
        tma_load_2d(dst + W_TILES * W_BYTES, &map_a, kx, 0, bar);
        issued = i + 1;
      }
      if (!ok) {
        atomicExch(error_flag, 1);
        // drain: every copy that was issued must land before the block may leave
        for (int i = max(0, issued - stages); i < issued; ++i) mbar_wait(full0 + 8 * (i % stages), (i / stages) & 1);
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NPAD >> 3) << 17) |
                             ((uint32_t)(kTileN >> 4) << 24);
      bool ok = true;
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % stages;
        ok = mbar_wait(full0 + 8 * s, (i / stages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t w_addr = smem_addr(smem + (size_t)s * STAGE_BYTES);
        const uint64_t w_desc = make_smem_desc(w_addr);
        const uint64_t a_desc = make_smem_desc(w_addr + W_TILES * W_BYTES);
#pragma unroll
        for (int k = 0; k < kTileK / 16; ++k) {
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          mma_bf16_ss(tmem_base, w_desc + 2 * k, a_desc + 2 * k, idesc, acc);
          if (MODE == MODE_SWIGLU)
            mma_bf16_ss(tmem_base + NPAD, make_smem_desc(w_addr + W_BYTES) + 2 * k, a_desc + 2 * k, idesc, acc);
        }
        mma_commit(empty0 + 8 * s);               // the stage is free once these MMAs have read it
      }
      if (!ok) atomicExch(error_flag, 2);
      mma_commit(done_bar);                       // accumulators complete (or nothing more will come)
    }
    __syncwarp();
  } else {
    // ----------------------------------------------------------- epilogue
    const int quarter = warp & 3;                 // TMEM lanes this warp may read
    // SWIGLU64: lanes 0-63 hold gate rows, lanes 64-127 the up rows of the same 64 outputs
    const int n = MODE == MODE_SWIGLU64 ? n0 + (quarter & 1) * 32 + lane : n0 + quarter * 32 + lane;
    const bool up_half = MODE == MODE_SWIGLU64 && quarter >= 2;
    pdl_wait();                                   // nothing is written before the kernel in front has finished
    // Rows that arrive pre-normed (x * w without the norm's row scale) get the scale here:
    // rsqrt(mean(x^2) + eps) from the per-chunk sums of squares the norm kernel left.
    __shared__ float row_scale[NPAD < 128 ? 128 : NPAD];
    if (row_sumsq != nullptr) {
      for (int m = threadIdx.x - 64; m < M; m += 128) {   // the 128 epilogue threads share the tokens
        float total = 0.0f;
        for (int c0 = 0; c0 < sumsq_chunks; c0 += 8) {              // 8 loads in flight, added in chunk order
          float part[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            part[j] = c0 + j < sumsq_chunks ? __ldcg(&row_sumsq[(size_t)m * sumsq_chunks + c0 + j]) : 0.0f;
#pragma unroll
          for (int j = 0; j < 8; ++j) total += part[j];
        }
        row_scale[m] = rsqrtf(total / (float)K + eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    bool ok = mbar_wait(done_bar, 0);
    if (!ok && lane == 0) atomicExch(error_flag, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float b = (MODE == MODE_STORE && bias != nullptr && n < N) ? bias[n] : 0.0f;
#pragma unroll
    for (int c = 0; c < NPAD; c += 16) {
      if (c >= M) break;                                         // uniform over the block
      uint32_t g[16], u[16];
      if (ok && num_kb > 0) {
        tmem_ld16(taddr + c, g);
        if (MODE == MODE_SWIGLU) tmem_ld16(taddr + NPAD + c, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0u;
      }
      if (MODE == MODE_SWIGLU64) {
        __shared__ float up_rows[64][17];                        // the up half of these 16 token columns
        if (up_half) {
#pragma unroll
          for (int j = 0; j < 16; ++j) up_rows[(quarter & 1) * 32 + lane][j] = __uint_as_float(g[j]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!up_half) {
#pragma unroll
          for (int j = 0; j < 16; ++j) u[j] = __float_as_uint(up_rows[(quarter & 1) * 32 + lane][j]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");         // read before the next round overwrites it
      }
      if (n < N && !up_half) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = c + j;
          if (m >= M) break;
          const float rs = row_sumsq != nullptr ? row_scale[m] : 1.0f;
          float v = __uint_as_float(g[j]) * rs;
          if (MODE == MODE_SWIGLU || MODE == MODE_SWIGLU64) {
            const float up = __uint_as_float(u[j]) * rs;
            v = __fdividef(v, 1.0f + __expf(-v)) * up;       // a few float32 ulps, far below the bfloat16 rounding
          }
          if (MODE == MODE_PARTIAL) {
            partials[((size_t)split * M + m) * N + n] = v;
          } else if (out_is_f32) {
            reinterpret_cast<float*>(out)[(size_t)m * N + n] = v + b;
          } else {
            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)m * N + n] = __float2bfloat16_rn(v + b);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------ host side

struct MapKey {
  const void* base;
  int rows, cols, box;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box == o.box; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (size_t)k.rows * 1000003u ^ (size_t)k.cols * 7919u ^ (size_t)k.box;
  }
};

// Weight maps are made once per weight tensor and kept.
static int weight_map(CUtensorMap* out, const void* base, int rows, int cols, int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  MapKey key{base, rows, cols, box_rows};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap m;
    int rc = make_tensor_map_bf16(&m, base, rows, cols, box_rows);
    if (rc) return rc;
    it = cache.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n <= 0)
      n = 148;
  }
  return n;
}

static size_t skinny_smem_bytes(int npad, int mode, int stages) {
  const size_t stage = (size_t)(mode == MODE_SWIGLU ? 2 : 1) * kTileN * kTileK * 2 + (size_t)npad * kTileK * 2;
  return 1024 + stages * stage + (2 * stages + 1) * 8 + 16;
}

template <int NPAD, int MODE>
static int launch_skinny(const CUtensorMap& mw, const CUtensorMap& ma, const float* bias, void* out, float* partials,
                         int M, int N, int K, int splits, int up_row_offset, int out_is_f32, const float* row_sumsq,
                         int sumsq_chunks, float eps, int* error_flag, cudaStream_t stream) {
  const int total_kblocks = (K + kTileK - 1) / kTileK;
  const int per_split = (total_kblocks + splits - 1) / splits;
  // As many stages as fit the block's share of shared memory, at most the k-blocks of a split.  A grid of at most
  // one block per SM gives every block the SM to itself; a larger one puts two on an SM so that all of them
  // stream at once and share the HBM rate evenly, whatever the grid's remainder (27,648 / 128 = 216 tiles of a
  // 32B-size gate/up product: 94 -> 83 us).  Blocks with 256 token rows (32 KB of activations a stage) own their SM.
  dim3 grid((N + (MODE == MODE_SWIGLU64 ? kTileN / 2 : kTileN) - 1) / (MODE == MODE_SWIGLU64 ? kTileN / 2 : kTileN), splits);
  const bool alone = NPAD == 256 || (long long)grid.x * grid.y <= sm_count();
  const size_t budget = alone ? 200 * 1024 : (MODE == MODE_SWIGLU ? 110 * 1024 : 100 * 1024);
  int stages = 8;
  while (stages > 2 && skinny_smem_bytes(NPAD, MODE, stages) > budget) --stages;
  if (stages > per_split) stages = per_split < 2 ? 2 : per_split;
  const size_t smem = skinny_smem_bytes(NPAD, MODE, stages);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NPAD, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return launch_pdl(gemm_skinny_kernel<NPAD, MODE>, grid, dim3(192), smem, stream, 1, mw, ma, bias, out, partials, M, N,
                    K, per_split, up_row_offset, out_is_f32, stages, row_sumsq, sumsq_chunks, eps, error_flag);
}

}  // namespace ifx

using namespace ifx;

// act [M, K] and W [rows, K] bfloat16, M <= 256, K % 8 == 0, both 16-byte aligned.
// mode 0: out[M, N] (+ bias) bfloat16 or float32, splits must be 1.
// mode 1: partials[splits, M, N] float32.
// mode 2: W holds N gate rows at 0 and N up rows at up_row_offset; out[M, N] = silu(gate) * up, bfloat16.
// error_flag: device int, set to non-zero if a bounded wait ran out (the output is then not valid).
// row_sumsq (optional): float32 [M, sumsq_chunks]; the rows of `act` are then x * w of a norm over K
// columns and every output row m is scaled by rsqrt(sum(row_sumsq[m, :]) / K + eps).
extern "C" int ifx_gemm_skinny(const void* act, const void* W, const float* bias, void* out, float* partials, int M,
                               int N, int K, int w_rows, int splits, int mode, int up_row_offset, int out_is_f32,
                               const float* row_sumsq, int sumsq_chunks, float eps, int* error_flag,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || M > 256 || splits <= 0 || splits > 65535 || error_flag == nullptr) return IFX_E_BADARG;
  if (mode == MODE_STORE && splits != 1) return IFX_E_BADARG;
  if (mode == MODE_SWIGLU && (splits != 1 || out_is_f32)) return IFX_E_BADARG;
  if (mode == MODE_PARTIAL && partials == nullptr) return IFX_E_BADARG;
  const int total_kblocks = (K + kTileK - 1) / kTileK;
  if (splits > total_kblocks) return IFX_E_BADARG;
  // a narrow gate/up product (at most half as many tiles as SMs): 64 + 64 weight rows a block
  if (mode == MODE_SWIGLU && 2 * ((N + kTileN - 1) / kTileN) <= sm_count()) mode = MODE_SWIGLU64;
  CUtensorMap mw, ma;
  int rc = weight_map(&mw, W, w_rows, K, mode == MODE_SWIGLU64 ? kTileN / 2 : kTileN);
  if (rc) return rc;
  const int npad = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
  rc = make_tensor_map_bf16(&ma, act, M, K, npad);
  if (rc) return rc;
#define LAUNCH(NP, MD) \
  return launch_skinny<NP, MD>(mw, ma, bias, out, partials, M, N, K, splits, up_row_offset, out_is_f32, row_sumsq, \
                               sumsq_chunks, eps, error_flag, stream)
#define BY_NPAD(MD)                 \
  switch (npad) {                   \
    case 16: LAUNCH(16, MD);        \
    case 32: LAUNCH(32, MD);        \
    case 64: LAUNCH(64, MD);        \
    case 128: LAUNCH(128, MD);      \
    default: LAUNCH(256, MD);       \
  }
  if (mode == MODE_STORE) { BY_NPAD(MODE_STORE) }
  if (mode == MODE_PARTIAL) { BY_NPAD(MODE_PARTIAL) }
  if (mode == MODE_SWIGLU) { BY_NPAD(MODE_SWIGLU) }
  if (mode == MODE_SWIGLU64) { BY_NPAD(MODE_SWIGLU64) }
  return IFX_E_BADARG;
}
