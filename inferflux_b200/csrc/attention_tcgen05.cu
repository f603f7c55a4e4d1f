// Attention of prompt portions on the 5th-generation tensor cores.
//
// A thread block takes up to 256 query tokens of one query head, as two tiles of 128, and
// walks the keys they may see in tiles of 128; both query tiles use each key/value tile that
// is fetched, which halves the traffic from L2.  Tensor memory holds, per query tile, the
// scores and the output:
//
//   S = Q . K^T     tcgen05.mma, M 128 (queries = TMEM lanes) x N 128 (keys), K = head size;
//                   Q and the key tile are K-major in shared memory (128-byte swizzle)
//   softmax         one group of four warps per query tile, one thread per query row: the row
//                   of S is read from TMEM (tcgen05.ld), masked on edge tiles, exponentiated
//                   against the row's reference maximum (log2 domain, one FFMA + one ex2 per
//                   score), and written back over S as bfloat16 pairs (tcgen05.st): the A
//                   operand of the next product
//   O += P . V      tcgen05.mma with A from tensor memory; V stays as the cache holds it
//                   (key-major rows), i.e. an MN-major B operand.  O accumulates in TMEM.
//
// The MMA warp alternates between the two query tiles, so that the tensor cores work on one
// tile while the other tile's softmax runs.  A reference maximum moves only when the running
// maximum has outgrown it by more than 2^8; then the thread rescales its row of O in TMEM.
// Probabilities therefore stay below 2^8, and sum and output are taken against the same
// reference, so the result is the softmax exactly (up to rounding).
//
// Warp 0 fetches: the query tiles once, then per key tile the pages of K and of V as TMA boxes
// [16 keys x 64 elements] through the block table, into a ring of slots (a slot holds the keys
// or the values of one tile).  Warp 1 issues the MMAs.  Warps 2-5 and 6-9 are the softmax groups.
//
// Keys outside a row's range get weight zero; what the cache holds there is finite (the pool
// starts as zeros and only finite values are written to it).  Page sizes: powers of two from
// 16; head sizes 64 and 128.  Every wait is bounded; a wait that runs out sets *error_flag.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ifx {

typedef __nv_bfloat16 bf16;

constexpr int kBM = 128;      // queries per block
constexpr int kBN = 128;      // keys per tile

__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t addr) {
  // rows of 128 bytes, 8-row groups 1024 bytes apart
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor_sw128(uint32_t addr, uint32_t atom_stride_bytes) {
  // 64 MN elements (128 bytes) contiguous, the next 64 `atom_stride_bytes` further; K rows 128 bytes
  // apart, 8-row groups 1024 bytes apart
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((atom_stride_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
  uint32_t* u = reinterpret_cast<uint32_t*>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
        "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
        "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
      : "r"(taddr));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&u)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31,%32};"
      ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]),
        "r"(u[9]), "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]),
        "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]),
        "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

constexpr float kRescaleStep = 8.0f;      // log2 units the maximum may outgrow its reference before O is rescaled
constexpr uint32_t kTmemCols = 512;       // per query tile: scores (128 columns) and output (head size)
constexpr int kThreads = 320;             // fetch warp, MMA warp, two softmax groups of four warps

template <int D>
struct PrefillLayout {
  static constexpr int HALVES = D / 64;                       // 64-element (128-byte) column blocks of a head
  static constexpr int SLOTS = D == 128 ? 5 : 8;              // key or value tiles in flight
  static constexpr uint32_t Q_BYTES = HALVES * kBM * 128;     // one query tile: [half][128 rows][128 B]
  static constexpr uint32_t SLOT_BYTES = HALVES * kBN * 128;  // the keys or the values of one tile
  static constexpr int B_Q = 0, B_FULL = 1, B_EMPTY = B_FULL + SLOTS, B_S_FULL = B_EMPTY + SLOTS,
                       B_P_FULL = B_S_FULL + 2, B_O_FULL = B_P_FULL + 2, B_COUNT = B_O_FULL + 2;
  static constexpr size_t SMEM = 1024 + 2 * Q_BYTES + (size_t)SLOTS * SLOT_BYTES + B_COUNT * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(kThreads)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap pool_map,
                            const int* __restrict__ block_table, const int* __restrict__ tiles,
                            const int* __restrict__ req_slot, bf16* __restrict__ out, int nq, int nkv, int page_size,
                            int page_shift, int max_blocks, int num_pages, int window, float scale_log2,
                            int* __restrict__ error_flag) {
  using L = PrefillLayout<D>;
  constexpr int HALVES = L::HALVES, SLOTS = L::SLOTS;
  constexpr uint32_t Q_BYTES = L::Q_BYTES, SLOT_BYTES = L::SLOT_BYTES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const uint32_t q_s = smem_addr(smem);                  // two query tiles
  const uint32_t kv_s = q_s + 2 * Q_BYTES;               // the ring of slots
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * Q_BYTES + SLOTS * SLOT_BYTES);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + L::B_COUNT);
  const uint32_t bar0 = smem_addr(bars);
  auto bar = [&](int i) { return bar0 + 8 * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    mbar_init(bar(L::B_Q), 1);
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(bar(L::B_FULL + s), 1);
      mbar_init(bar(L::B_EMPTY + s), 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(bar(L::B_S_FULL + q), 1);
      mbar_init(bar(L::B_P_FULL + q), 4);
      mbar_init(bar(L::B_O_FULL + q), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_holder)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * kBN;       // S of tile q: + q * 128; O: + q * D
  pdl_wait();

  // the last items of a prompt see the most keys: they go first; the heads of an item run side by side
  const int* tile = tiles + (size_t)(gridDim.y - 1 - blockIdx.y) * 4;
  const int r = tile[0], row0 = tile[1], rows = tile[2], pos0 = tile[3];
  const int h = blockIdx.x;
  const int g = h / (nq / nkv);
  // key tiles [tb_q, te_q) of query tile q (rows q * 128 ...); tile 1 may be absent
  const int rows_1 = max(rows - kBM, 0);
  const int tb_0 = (window > 0 ? max(0, pos0 - window + 1) : 0) / kBN;
  const int te_0 = (pos0 + min(rows, kBM) + kBN - 1) / kBN;
  const int tb_1 = (window > 0 ? max(0, pos0 + kBM - window + 1) : 0) / kBN;
  const int te_1 = rows_1 > 0 ? (pos0 + rows + kBN - 1) / kBN : tb_1;
  const int tb = tb_0, te = max(te_0, te_1);
  const int kfirst = window > 0 ? max(0, pos0 - window + 1) : 0, kend = pos0 + rows;

  if (warp == 0) {
    // ------------------------------------------------------------------ fetching
    const int* table = block_table + (size_t)req_slot[r] * max_blocks;
    if (lane == 0) {
      mbar_expect_tx(bar(L::B_Q), rows_1 > 0 ? 2 * Q_BYTES : Q_BYTES);
      for (int q = 0; q < (rows_1 > 0 ? 2 : 1); ++q)
#pragma unroll
        for (int hh = 0; hh < HALVES; ++hh)
          tma_load_2d(q_s + q * Q_BYTES + hh * kBM * 128, &q_map, h * D + hh * 64, row0 + q * kBM, bar(L::B_Q));
    }
    bool ok = true;
    int issued = 0;                                       // slots filled so far
    for (int kt = tb; kt < te && ok; ++kt) {
      // lanes 0-7 take one 16-key block each; its page is looked up before the wait for a free slot
      const int key = kt * kBN + lane * 16;
      int page = 0, off = 0;
      if (lane < kBN / 16 && key < kend && key + 16 > kfirst) {      // else: any valid page, its keys get weight zero
        page = table[key >> page_shift];
        if (page < 0 || page >= num_pages) page = 0;
        off = key & (page_size - 1);
      }
#pragma unroll 1
      for (int kv = 0; kv < 2; ++kv) {                     // the keys, then the values
        const int j = 2 * (kt - tb) + kv, s = j % SLOTS;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::B_EMPTY + s), ((j / SLOTS) & 1) ^ 1));
        if (!ok) break;
        const uint32_t fb = bar(L::B_FULL + s);
        if (lane == 0) mbar_expect_tx(fb, SLOT_BYTES);
        __syncwarp();
        if (lane < kBN / 16) {
          const uint32_t dst = kv_s + s * SLOT_BYTES + lane * 2048;
          const int y = ((page * 2 + kv) * nkv + g) * page_size + off;
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh) tma_load_2d(dst + hh * kBN * 128, &pool_map, hh * 64, y, fb);
        }
        issued = j + 1;
      }
    }
    if (!ok && lane == 0) {
      atomicExch(error_flag, 7);
      for (int j = max(0, issued - SLOTS); j < issued; ++j)        // let the copies in flight land
        mbar_wait(bar(L::B_FULL + j % SLOTS), (j / SLOTS) & 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) |
                               ((uint32_t)(kBM >> 4) << 24);                       // both operands K-major
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) |
                               ((uint32_t)(kBM >> 4) << 24);                       // B (values) MN-major
      auto active = [&](int q, int kt) { return q == 0 ? (kt >= tb_0 && kt < te_0) : (kt >= tb_1 && kt < te_1); };
      auto last_q = [&](int kt) { return active(1, kt) ? 1 : 0; };    // the query tile that uses a key tile last
      bool ok = mbar_wait(bar(L::B_Q), 0);
      auto issue_s = [&](int q, int kt) -> bool {         // S_q = Q_q . K(kt)^T
        const int j = 2 * (kt - tb), s = j % SLOTS;
        if (!mbar_wait(bar(L::B_FULL + s), (j / SLOTS) & 1)) return false;
        tc_fence_after();
        const uint32_t k_src = kv_s + s * SLOT_BYTES, q_src = q_s + q * Q_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t half = k / 4, inner = (k % 4) * 32;
          umma_bf16(tmem_s + q * kBN, desc_kmajor_sw128(q_src + half * kBM * 128) + (inner >> 4),
                    desc_kmajor_sw128(k_src + half * kBN * 128) + (inner >> 4), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(bar(L::B_S_FULL + q));
        if (q == last_q(kt)) umma_commit(bar(L::B_EMPTY + s));      // the keys have been read
        return true;
      };
      int done[2] = {0, 0};                                // key tiles of each query tile so far
      auto issue_pv = [&](int q, int kt) -> bool {        // O_q += P_q . V(kt)
        const int j = 2 * (kt - tb) + 1, s = j % SLOTS;
        if (!mbar_wait(bar(L::B_P_FULL + q), done[q] & 1) || !mbar_wait(bar(L::B_FULL + s), (j / SLOTS) & 1))
          return false;
        tc_fence_after();
        const uint32_t v_src = kv_s + s * SLOT_BYTES;
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k)                 // 16 keys (8 columns of pairs) a step
          umma_bf16_ts(tmem_o + q * D, tmem_s + q * kBN + k * 8, desc_mnmajor_sw128(v_src + k * 2048, kBN * 128),
                       idesc_o, (done[q] > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar(L::B_O_FULL + q));
        if (q == last_q(kt)) umma_commit(bar(L::B_EMPTY + s));      // the values have been read
        ++done[q];
        return true;
      };
      for (int q = 0; q < 2 && ok; ++q)
        if (active(q, tb)) ok = issue_s(q, tb);
      for (int kt = tb; kt < te && ok; ++kt) {
        for (int q = 0; q < 2 && ok; ++q) {
          if (!active(q, kt)) continue;
          if (kt != tb && kt == (q == 0 ? tb_0 : tb_1)) ok = issue_s(q, kt);   // a tile that starts later (window)
          if (ok) ok = issue_pv(q, kt);
          // the next scores of this query tile go over its probabilities: the product that reads them
          // was issued just before and runs first; meanwhile the other tile's softmax is at work
          if (ok && active(q, kt + 1)) ok = issue_s(q, kt + 1);
        }
      }
      if (!ok) atomicExch(error_flag, 8);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax: one query tile, one row per thread
    const int q = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // TMEM lane = query row of the tile
    const int rows_q = q == 0 ? min(rows, kBM) : rows_1;
    const int pos0_q = pos0 + q * kBM;
    const int pos = pos0_q + row;
    const int wfirst = window > 0 ? pos - window + 1 : 0;
    const int tb_q = q == 0 ? tb_0 : tb_1, te_q = q == 0 ? te_0 : te_1;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem_s + q * kBN + lane_addr, o_addr = tmem_o + q * D + lane_addr;
    float m_ref = -INFINITY, l_run = 0.0f;
    bool ok = true;
    int i = 0;
    for (int kt = tb_q; kt < te_q; ++kt, ++i) {
      const int key0 = kt * kBN;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(L::B_S_FULL + q), i & 1));
      if (!ok) break;
      tc_fence_after();
      const bool edge = key0 + kBN - 1 > pos0_q || (window > 0 && key0 < pos0_q + kBM - window);
      // pass 1: the row's maximum
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kBN; c += 64) {
        float s[64];
        tmem_ld32(s_addr + c, *reinterpret_cast<float(*)[32]>(&s[0]));
        tmem_ld32(s_addr + c + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
        tmem_wait_ld();
        if (edge) {
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int key = key0 + c + j;
            if (key > pos || key < wfirst) s[j] = -INFINITY;
          }
        }
#pragma unroll
        for (int j = 0; j < 64; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the reference maximum moves only when the row's maximum has outgrown it
      const bool outgrown = m_ref > -INFINITY && (mx - m_ref) * scale_log2 > kRescaleStep;
      float factor = 1.0f;
      if (outgrown) {
        factor = ex2((m_ref - mx) * scale_log2);
        m_ref = mx;
        l_run *= factor;
      } else if (m_ref == -INFINITY) {
        m_ref = mx;                                        // nothing accumulated for this row so far
      }
      if (i > 0 && __any_sync(0xffffffffu, outgrown)) {    // rescale this warp's rows of O in tensor memory
        ok = __all_sync(0xffffffffu, mbar_wait(bar(L::B_O_FULL + q), (i - 1) & 1));   // the products so far are done
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          float t[32];
          tmem_ld32(o_addr + c, t);
          tmem_wait_ld();
          uint32_t u[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) u[j] = __float_as_uint(t[j] * factor);
          tmem_st32(o_addr + c, u);
        }
        tmem_wait_st();
      }
      // pass 2: probabilities over the scores, 64 keys (32 columns of bfloat16 pairs) at a time
      const float bias = m_ref == -INFINITY ? 0.0f : -m_ref * scale_log2;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < kBN; c += 64) {
        float s[64];
        tmem_ld32(s_addr + c, *reinterpret_cast<float(*)[32]>(&s[0]));
        tmem_ld32(s_addr + c + 32, *reinterpret_cast<float(*)[32]>(&s[32]));
        tmem_wait_ld();
        if (edge) {
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            const int key = key0 + c + j;
            if (key > pos || key < wfirst) s[j] = -INFINITY;
          }
        }
        uint32_t packed[32];
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          const float p0 = ex2(fmaf(s[j], scale_log2, bias));
          const float p1 = ex2(fmaf(s[j + 1], scale_log2, bias));
          sum4[(j >> 1) & 3] += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          packed[j >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        tmem_st32(s_addr + (c >> 1), packed);              // columns whose scores have been read already
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(L::B_P_FULL + q));
    }
    if (ok && i > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar(L::B_O_FULL + q), (i - 1) & 1));
    if (!ok && lane == 0) atomicExch(error_flag, 9);
    if (ok && i > 0) {
      tc_fence_after();
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      bf16* dst = out + ((size_t)(row0 + q * kBM + row) * nq + h) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        float t[32];
        tmem_ld32(o_addr + c, t);
        tmem_wait_ld();
        if (row < rows_q) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) v2[e] = __floats2bfloat162_rn(t[j + 2 * e] * inv, t[j + 2 * e + 1] * inv);
            *reinterpret_cast<uint4*>(dst + c + j) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <int D>
static int launch_prefill_tcgen05(const bf16* q, int num_tokens, const bf16* kv_pool, const int* block_table,
                                  const int* tiles, const int* req_slot, bf16* out, int num_tiles, int nq, int nkv,
                                  int page_size, int page_shift, int max_blocks, int num_pages, int window,
                                  float scale_log2, int* error_flag, cudaStream_t stream) {
  CUtensorMap q_map, pool_map;
  int rc = make_tensor_map_bf16(&q_map, q, num_tokens, nq * D, kBM);
  if (rc) return rc;
  rc = pool_tensor_map(&pool_map, kv_pool, (long long)num_pages * 2 * nkv * page_size, D);
  if (rc) return rc;
  const size_t smem = PrefillLayout<D>::SMEM;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(attn_prefill_tcgen05_kernel<D>, dim3(nq, num_tiles), dim3(kThreads), smem, stream, 1, q_map,
                    pool_map, block_table, tiles, req_slot, out, nq, nkv, page_size, page_shift, max_blocks,
                    num_pages, window, scale_log2, error_flag);
}

}  // namespace ifx

using namespace ifx;

extern "C" {

// 1 if the tensor-core kernel takes this head size and page size.
int ifx_attention_prefill_tcgen05_supports(int d, int page_size) {
  return (d == 64 || d == 128) && page_size >= 16 && (page_size & (page_size - 1)) == 0;
}

// q [num_tokens, nq * d] bfloat16, 16-byte aligned.  tiles: int32 [num_tiles, 4] = (request index, first
// flat row, rows <= 256, first position).
int ifx_attention_prefill_tcgen05(const void* q, int num_tokens, const void* kv_pool, const int* block_table,
                                  const int* tiles, const int* req_slot, void* out, int num_tiles, int nq, int nkv,
                                  int d, int page_size, int max_blocks, int num_pages, int window, float scale,
                                  int* error_flag, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (!ifx_attention_prefill_tcgen05_supports(d, page_size) || nq <= 0 || nkv <= 0 || nq % nkv || max_blocks <= 0 ||
      num_tiles > 65535 || !(scale > 0.0f) || error_flag == nullptr)
    return IFX_E_BADARG;
  int ps = 0;
  while ((1 << ps) < page_size) ++ps;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (d == 64)
    return launch_prefill_tcgen05<64>((const bf16*)q, num_tokens, (const bf16*)kv_pool, block_table, tiles, req_slot,
                                      (bf16*)out, num_tiles, nq, nkv, page_size, ps, max_blocks, num_pages, window,
                                      scale_log2, error_flag, stream);
  return launch_prefill_tcgen05<128>((const bf16*)q, num_tokens, (const bf16*)kv_pool, block_table, tiles, req_slot,
                                     (bf16*)out, num_tiles, nq, nkv, page_size, ps, max_blocks, num_pages, window,
                                     scale_log2, error_flag, stream);
}

}  // extern "C"
