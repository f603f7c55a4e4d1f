// Matrix product for many token rows (prompt portions) on the 5th-generation tensor cores:
// out[M, N] = act[M, K] . W[N, K]^T, bfloat16 in, float32 accumulation in tensor memory, with
// the epilogues a decoder layer wants fused in:
//
//   STORE    out[m, n] = acc                                   (bfloat16)
//   SWIGLU   W holds N gate rows and, `up_row_offset` rows further, N up rows;
//            out[m, n] = silu(acc_gate) * acc_up               (bfloat16; no [M, 2N] round trip,
//                                                               no separate activation kernel)
//
// A persistent grid of one block per SM walks the output tiles of 128 token rows x 256 weight
// rows (SWIGLU: 128 gate + 128 up rows of the same 128 outputs), token tiles fastest, so that
// the blocks running at a time share a few weight panels in L2.  Per block:
//
//   warp 0     producer: TMA (cp.async.bulk.tensor, 128-byte swizzle) of the activation tile
//              [128 x 64] and the weight tile [256 x 64] of every k-block into a ring of four
//              48 KB stages, each guarded by a full/empty mbarrier;
//   warp 1     issues tcgen05.mma (cta_group::1, kind::f16, M 128, N 256, K 16) into one of two
//              256-column accumulators in tensor memory; tcgen05.commit frees a stage, and hands
//              a finished accumulator to the epilogue;
//   warps 2-5  epilogue: tcgen05.ld of their 32 token rows, 16 columns at a time, conversion (and
//              SiLU * up), 32-byte stores; it runs under the products of the next tile.
//
// No TMA multicast, no thread-block clusters.  Every wait on an mbarrier is bounded: a wait that
// runs out sets *error_flag and the block winds down (drains its copies, frees its tensor memory).
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ifx {

constexpr int kBM = 128, kBN = 256, kBK = 64, kGemmStages = 4;
constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = kBN * kBK * 2, kStageBytes = kABytes + kBBytes;

enum { GEMM_STORE = 0, GEMM_SWIGLU = 1 };

__device__ __forceinline__ uint64_t gemm_smem_desc(uint32_t addr) {
  // K-major tile of 128-byte rows, 128-byte swizzle: 8-row groups 1024 bytes apart.
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
__device__ __forceinline__ void gemm_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void gemm_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void gemm_tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void gemm_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int MODE>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    __nv_bfloat16* __restrict__ out, int M, int N, int K, int up_row_offset, int m_tiles, int n_tiles,
                    int* __restrict__ error_flag) {
  constexpr int OUT_COLS = MODE == GEMM_SWIGLU ? kBN / 2 : kBN;     // output columns a tile makes
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)kGemmStages * kStageBytes);
  // full[4], empty[4], acc_full[2], acc_empty[2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kGemmStages + 4);
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + kGemmStages);
  const uint32_t acc_full0 = smem_addr(bars + 2 * kGemmStages), acc_empty0 = smem_addr(bars + 2 * kGemmStages + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = m_tiles * n_tiles;
  const int kblocks = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_holder)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int idx = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * kBM, n0 = (t / m_tiles) * OUT_COLS;
        for (int kb = 0; kb < kblocks; ++kb, ++idx) {
          const int s = idx % kGemmStages;
          if (idx >= kGemmStages) ok = mbar_wait(empty0 + 8 * s, ((idx / kGemmStages) & 1) ^ 1);
          if (!ok) break;
          const uint32_t dst = smem_addr(smem + (size_t)s * kStageBytes), bar = full0 + 8 * s;
          mbar_expect_tx(bar, kStageBytes);
          tma_load_2d(dst, &map_a, kb * kBK, m0, bar);
          if (MODE == GEMM_SWIGLU) {
            tma_load_2d(dst + kABytes, &map_w, kb * kBK, n0, bar);                       // 128 gate rows
            tma_load_2d(dst + kABytes + kBBytes / 2, &map_w, kb * kBK, up_row_offset + n0, bar);   // 128 up rows
          } else {
            tma_load_2d(dst + kABytes, &map_w, kb * kBK, n0, bar);
            tma_load_2d(dst + kABytes + kBBytes / 2, &map_w, kb * kBK, n0 + 128, bar);
          }
        }
      }
      if (!ok) {
        atomicExch(error_flag, 21);
        for (int i = max(0, idx - kGemmStages); i < idx; ++i) mbar_wait(full0 + 8 * (i % kGemmStages), (i / kGemmStages) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      int idx = 0, tile = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile) {
        const int buf = tile & 1, use = tile >> 1;
        if (use > 0) ok = mbar_wait(acc_empty0 + 8 * buf, (use & 1) ^ 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * kBN;
        for (int kb = 0; kb < kblocks; ++kb, ++idx) {
          const int s = idx % kGemmStages;
          ok = mbar_wait(full0 + 8 * s, (idx / kGemmStages) & 1);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_addr(smem + (size_t)s * kStageBytes);
          const uint64_t a_desc = gemm_smem_desc(a_addr), b_desc = gemm_smem_desc(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) gemm_mma(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          gemm_commit(empty0 + 8 * s);
        }
        if (ok) gemm_commit(acc_full0 + 8 * buf);
      }
      if (!ok) atomicExch(error_flag, 22);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                                     // TMEM lanes (token rows) of this warp
    int tile = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile) {
      const int buf = tile & 1, use = tile >> 1;
      const int m = (t % m_tiles) * kBM + quarter * 32 + lane, n0 = (t / m_tiles) * OUT_COLS;
      ok = mbar_wait(acc_full0 + 8 * buf, use & 1);
      if (!ok) {
        if (lane == 0) atomicExch(error_flag, 23);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kBN;
      __nv_bfloat16* row = out + (size_t)m * N + n0;
      const bool vec = (N % 8) == 0;                                  // rows start on 16-byte boundaries
#pragma unroll 2
      for (int c = 0; c < OUT_COLS; c += 16) {
        uint32_t g[16], u[16];
        gemm_tmem_ld16(taddr + c, g);
        if (MODE == GEMM_SWIGLU) gemm_tmem_ld16(taddr + kBN / 2 + c, u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          v[j] = __uint_as_float(g[j]);
          if (MODE == GEMM_SWIGLU) v[j] = __fdividef(v[j], 1.0f + __expf(-v[j])) * __uint_as_float(u[j]);
        }
        if (m < M) {
          if (vec && n0 + c + 16 <= N) {
            uint4 lo = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            uint4 hi = make_uint4(pack_bf16(v[8], v[9]), pack_bf16(v[10], v[11]), pack_bf16(v[12], v[13]), pack_bf16(v[14], v[15]));
            *reinterpret_cast<uint4*>(row + c) = lo;
            *reinterpret_cast<uint4*>(row + c + 8) = hi;
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (n0 + c + j < N) row[c + j] = __float2bfloat16_rn(v[j]);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) gemm_mbar_arrive(acc_empty0 + 8 * buf);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

static int gemm_sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 1;
  }
  return sms;
}

template <int MODE>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mw, void* out, int M, int N, int K, int up_row_offset,
                       int* error_flag, cudaStream_t stream) {
  constexpr int OUT_COLS = MODE == GEMM_SWIGLU ? kBN / 2 : kBN;
  const size_t smem = 1024 + (size_t)kGemmStages * kStageBytes + (2 * kGemmStages + 4) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + OUT_COLS - 1) / OUT_COLS;
  const int tiles = m_tiles * n_tiles;
  const int grid = tiles < gemm_sm_count() ? tiles : gemm_sm_count();
  gemm_tcgen05_kernel<MODE><<<grid, 192, smem, stream>>>(ma, mw, reinterpret_cast<__nv_bfloat16*>(out), M, N, K,
                                                         up_row_offset, m_tiles, n_tiles, error_flag);
  IFX_CHECK_LAUNCH();
  return 0;
}

}  // namespace ifx

using namespace ifx;

// act [M, K] and W [w_rows, K] bfloat16, K % 8 == 0, both 16-byte aligned; out [M, N] bfloat16.
// mode 0: out = act . W[:N]^T.   mode 1: out = silu(act . W[:N]^T) * (act . W[up_row_offset : up_row_offset + N]^T).
// error_flag: device int, set to non-zero if a bounded wait ran out (the output is then not valid).
extern "C" int ifx_gemm_tcgen05(const void* act, const void* W, void* out, int M, int N, int K, int w_rows, int mode,
                                int up_row_offset, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || error_flag == nullptr || out == nullptr) return IFX_E_BADARG;
  if (mode == GEMM_SWIGLU && (up_row_offset < N || up_row_offset + N > w_rows)) return IFX_E_BADARG;
  if (mode == GEMM_STORE && N > w_rows) return IFX_E_BADARG;
  CUtensorMap ma, mw;
  int rc = weight_tensor_map(&mw, W, w_rows, K, 128);
  if (rc) return rc;
  rc = make_tensor_map_bf16(&ma, act, M, K, kBM);
  if (rc) return rc;
  if (mode == GEMM_STORE) return launch_gemm<GEMM_STORE>(ma, mw, out, M, N, K, 0, error_flag, stream);
  if (mode == GEMM_SWIGLU) return launch_gemm<GEMM_SWIGLU>(ma, mw, out, M, N, K, up_row_offset, error_flag, stream);
  return IFX_E_BADARG;
}
