// Tiled bfloat16 attention over the paged cache on the warp-level tensor-core path
// (mma.sync m16n8k16, ldmatrix, cp.async): one kernel for prompt portions and one,
// with the key range split over thread blocks, for single decoded tokens.
//
// Both read keys and values through the block table, page by page, into shared
// memory whose rows are padded by 16 bytes so that ldmatrix reads are free of bank
// conflicts.  Scores, the running maximum and sum, and the output accumulate in
// float32; the softmax works in the log2 domain (scores are multiplied by
// scale * log2(e) once, then exp2f).
//
// Prompt portions: a thread block takes a tile of up to 64 query tokens of one
// query head; each of its 4 warps owns 16 query rows; key/value tiles of 64 keys
// are double-buffered.  The keys a row may see are [max(0, pos - window + 1), pos].
//
// Decoded tokens: a thread block takes one token, one key/value head and one
// split of the key range.  The query heads that share the key/value head (up to
// 16) are the 16 rows of the MMA tile, so every key and value is read once for all
// of them.  Each warp walks its own 16-key tiles through a 3-stage cp.async
// pipeline; the warps' partial results are merged in shared memory.  When the key
// range is split, the blocks of one (token, key/value head) form a thread-block
// cluster (up to 8): after a cluster barrier each block merges its share of the
// head dimensions from all blocks' shared memory (distributed shared memory), in
// block order - no scratch in global memory, no second kernel, nothing spins.
// Both kernels copy the block-table entries of their key range to shared memory
// first, so that page lookups do not sit on the critical path of the loads.
//
// Head sizes: 16, 32, 48, 64, 80, 96, 112, 128 and 256.  Others, and query groups
// larger than 16 in decoding, are refused (the caller then uses the generic kernel).
#include <cooperative_groups.h>

#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace ifx {

namespace cg = cooperative_groups;
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x in one MUFU instruction (flushes denormal results to zero, which is what a softmax weight
// that small should be); ex2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct PageMap {
  const int* table;      // this request's row of the block table, or a shared-memory copy of a part of it
  int blk_base;          // the logical block that table[0] stands for
  int page_size, page_shift, num_pages, nkv, g;
  // Element offset of key `k`'s row (head g) in the pool; the value row lies v_off further.
  __device__ __forceinline__ size_t key_row(int k, int d) const {
    int blk, off;
    if (page_shift >= 0) {
      blk = k >> page_shift;
      off = k & (page_size - 1);
    } else {
      blk = k / page_size;
      off = k - blk * page_size;
    }
    int page = table[blk - blk_base];
    if (page < 0 || page >= num_pages) page = 0;          // a broken table must not leave the pool
    return ((((size_t)page * 2) * nkv + g) * page_size + off) * d;
  }
};

// ------------------------------------------------------------- prompt portions
template <int D, int KT>
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv_pool, const int* __restrict__ block_table,
                    const int* __restrict__ tiles, const int* __restrict__ req_slot, bf16* __restrict__ out, int nq,
                    int nkv, int page_size, int page_shift, int max_blocks, int num_pages, int window,
                    float scale_log2, int tbl_cap) {
  constexpr int LDS = D + 8;            // shared-memory row stride in elements
  constexpr int CPR = D / 8;            // 16-byte chunks per row
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);        // [64][LDS]
  bf16* k_s = q_s + 64 * LDS;                           // [2][KT][LDS]
  bf16* v_s = k_s + 2 * KT * LDS;                       // [2][KT][LDS]
  int* tbl_s = reinterpret_cast<int*>(v_s + 2 * KT * LDS);   // [tbl_cap] block-table entries of this tile's keys

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* tile = tiles + (size_t)(blockIdx.x >> 2) * 4;   // a work item has up to 256 rows: four blocks
  const int half = (blockIdx.x & 3) * 64;
  if (tile[2] <= half) return;
  const int r = tile[0], row0 = tile[1] + half, rows = min(64, tile[2] - half), pos0 = tile[3] + half;
  const int h = blockIdx.y;
  const int* table_g = block_table + (size_t)req_slot[r] * max_blocks;
  PageMap pm{table_g, 0, page_size, page_shift, num_pages, nkv, h / (nq / nkv)};
  const size_t v_off = (size_t)nkv * page_size * D;

  const int kfirst = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kend = pos0 + rows;
  const int tile_begin = kfirst / KT, tile_end = (kend + KT - 1) / KT;
  {   // the block-table entries of keys [kfirst, kend) go to shared memory once
    const int b0 = kfirst / page_size, b1 = (kend - 1) / page_size;
    if (b1 - b0 + 1 <= tbl_cap) {
      for (int i = tid; i <= b1 - b0; i += 128) tbl_s[i] = table_g[b0 + i];
      pm.table = tbl_s;
      pm.blk_base = b0;
      __syncthreads();
    }
  }

  for (int i = tid; i < 64 * CPR; i += 128) {
    const int row = i / CPR, c = i % CPR;
    bf16* dst = q_s + row * LDS + c * 8;
    if (row < rows)
      cp_async16(smem_u32(dst), q + ((size_t)(row0 + row) * nq + h) * D + c * 8);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
  auto load_tile = [&](int t, int stage) {
    for (int i = tid; i < KT * CPR; i += 128) {
      const int row = i / CPR, c = i % CPR;
      const int k = t * KT + row;
      bf16* kd = k_s + (stage * KT + row) * LDS + c * 8;
      bf16* vd = v_s + (stage * KT + row) * LDS + c * 8;
      if (k >= kfirst && k < kend) {
        const bf16* src = kv_pool + pm.key_row(k, D) + c * 8;
        cp_async16(smem_u32(kd), src);
        cp_async16(smem_u32(vd), src + v_off);
      } else {                                              // never multiply by whatever lies there
        *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  load_tile(tile_begin, 0);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  const int p_lo = pos0 + warp * 16 + (lane >> 2), p_hi = p_lo + 8;
  const int w_lo = window > 0 ? p_lo - window + 1 : 0, w_hi = window > 0 ? p_hi - window + 1 : 0;

  for (int t = tile_begin; t < tile_end; ++t) {
    const int stage = (t - tile_begin) & 1;
    if (t + 1 < tile_end) load_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (t == tile_begin) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, col = kk * 16 + (lane >> 4) * 8;
        ldmatrix_x4(qf[kk], smem_u32(q_s + row * LDS + col));
      }
    }
    const bf16* kt = k_s + stage * KT * LDS;
    const bf16* vt = v_s + stage * KT * LDS;
    float s[KT / 8][4];
#pragma unroll
    for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < KT / 16; ++n2) {
        uint32_t b[4];
        const int row = n2 * 16 + (lane >> 4) * 8 + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b, smem_u32(kt + row * LDS + col));
        mma_bf16(s[2 * n2], qf[kk], b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], qf[kk], b[2], b[3]);
      }
    }
    // Masking only where a key of the tile can be invisible to a row of this warp: a tile that lies
    // wholly inside every row's range (most tiles of a long prompt) skips the compares.
    const int key0 = t * KT;
    const bool inside = key0 + KT - 1 <= pos0 + warp * 16 && key0 >= kfirst &&
                        (window <= 0 || key0 >= pos0 + warp * 16 + 15 - window + 1);
    if (!inside) {
#pragma unroll
      for (int n = 0; n < KT / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + n * 8 + 2 * (lane & 3) + (e & 1);
          const bool ok = e < 2 ? (key <= p_lo && key >= w_lo) : (key <= p_hi && key >= w_hi);
          if (!ok) s[n][e] = -INFINITY;
        }
      }
    }
    // running maximum of the raw scores; the scale (positive) goes into the exponent's multiply-add
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < KT / 8; ++n) {
      mx_lo = fmaxf(mx_lo, fmaxf(s[n][0], s[n][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[n][2], s[n][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    const float mu_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, mu_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
    const float c_lo = fast_exp2((m_lo - mu_lo) * scale_log2), c_hi = fast_exp2((m_hi - mu_hi) * scale_log2);
    const float b_lo = -mu_lo * scale_log2, b_hi = -mu_hi * scale_log2;
    m_lo = mn_lo;
    m_hi = mn_hi;
    l_lo *= c_lo;
    l_hi *= c_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= c_lo;
      o[i][1] *= c_lo;
      o[i][2] *= c_hi;
      o[i][3] *= c_hi;
    }
    uint32_t pa[KT / 16][4];
#pragma unroll
    for (int n = 0; n < KT / 8; ++n) {
      const float e0 = fast_exp2(fmaf(s[n][0], scale_log2, b_lo)), e1 = fast_exp2(fmaf(s[n][1], scale_log2, b_lo));
      const float e2 = fast_exp2(fmaf(s[n][2], scale_log2, b_hi)), e3 = fast_exp2(fmaf(s[n][3], scale_log2, b_hi));
      l_lo += e0 + e1;
      l_hi += e2 + e3;
      pa[n >> 1][(n & 1) * 2] = pack_bf16(e0, e1);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(e2, e3);
    }
#pragma unroll
    for (int j = 0; j < KT / 16; ++j) {
#pragma unroll
      for (int d2 = 0; d2 < D / 16; ++d2) {
        uint32_t b[4];
        const int row = j * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = d2 * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(b, smem_u32(vt + row * LDS + col));
        mma_bf16(o[2 * d2], pa[j], b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], pa[j], b[2], b[3]);
      }
    }
    __syncthreads();
  }
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float i_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, i_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int col = n * 8 + 2 * (lane & 3);
    if (r_lo < rows)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_lo) * nq + h) * D + col) =
          pack_bf16(o[n][0] * i_lo, o[n][1] * i_lo);
    if (r_hi < rows)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r_hi) * nq + h) * D + col) =
          pack_bf16(o[n][2] * i_hi, o[n][3] * i_hi);
  }
}

// -------------------------------------------------------------- decoded tokens
template <int D, int STAGES>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv_pool, const int* __restrict__ block_table,
                   const int4* __restrict__ decode_meta, bf16* __restrict__ out, int nq, int nkv, int page_size,
                   int page_shift, int max_blocks, int num_pages, int window, float scale_log2, int tbl_cap) {
  constexpr int LDS = D + 8;
  constexpr int CPR = D / 8;
  constexpr int STAGE_ELEMS = 2 * 16 * LDS;             // K tile then V tile
  constexpr int STAGE_BYTES_ALL = 4 * STAGES * STAGE_ELEMS * 2;
  constexpr int MERGE_BYTES = (4 * 16 * D + 2 * 4 * 16) * 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);        // [16][LDS]
  bf16* stage_base = q_s + 16 * LDS;                    // [4 warps][STAGES][2][16][LDS]
  constexpr int FIN_BYTES = (16 * D + 32) * 4;
  constexpr int WORK_BYTES = STAGE_BYTES_ALL > MERGE_BYTES + FIN_BYTES ? STAGE_BYTES_ALL : MERGE_BYTES + FIN_BYTES;
  // the block's merged result lives behind the warps' merge buffers, inside the (by then free) staging area
  float* fin_o = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(stage_base) + MERGE_BYTES);   // [16][D]
  float* fin_m = fin_o + 16 * D;                        // [16] this block's maximum per row (log2 domain)
  float* fin_l = fin_m + 16;                            // [16] this block's sum per row
  int* tbl_s = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(stage_base) + WORK_BYTES);   // [tbl_cap]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int item = blockIdx.x, g = blockIdx.y, split = blockIdx.z, num_splits = gridDim.z;
  const int G = nq / nkv;
  const int4 meta = decode_meta[item];                  // (flat token row, position, request slot, -)
  const int t = meta.x;
  const int pos = meta.y;
  const int* table_g = block_table + (size_t)meta.z * max_blocks;
  PageMap pm{table_g, 0, page_size, page_shift, num_pages, nkv, g};
  const size_t v_off = (size_t)nkv * page_size * D;

  const int kfirst = window > 0 ? max(0, pos - window + 1) : 0;
  const int kend = pos + 1;
  const int per_split = (((kend - kfirst + num_splits - 1) / num_splits) + 63) / 64 * 64;
  const int k0 = kfirst + split * per_split;
  const int k1 = min(kend, k0 + per_split);
  if (k0 < k1) {   // the block-table entries of keys [k0, k1) go to shared memory once
    const int b0 = k0 / page_size, b1 = (k1 - 1) / page_size;
    if (b1 - b0 + 1 <= tbl_cap) {
      for (int i = tid; i <= b1 - b0; i += 128) tbl_s[i] = table_g[b0 + i];
      pm.table = tbl_s;
      pm.blk_base = b0;
    }
  }

  for (int i = tid; i < 16 * CPR; i += 128) {
    const int row = i / CPR, c = i % CPR;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < G) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * nq + g * G + row) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + row * LDS + c * 8) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8, col = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[kk], smem_u32(q_s + row * LDS + col));
  }

  bf16* my_stages = stage_base + (size_t)warp * STAGES * STAGE_ELEMS;
  auto load_tile = [&](int base, int stage) {            // keys base .. base + 15 of this warp
    bf16* kd0 = my_stages + stage * STAGE_ELEMS;
    for (int i = lane; i < 16 * CPR; i += 32) {
      const int row = i / CPR, c = i % CPR;
      const int k = base + row;
      bf16* kd = kd0 + row * LDS + c * 8;
      bf16* vd = kd + 16 * LDS;
      if (k < k1) {
        const bf16* src = kv_pool + pm.key_row(k, D) + c * 8;
        cp_async16(smem_u32(kd), src);
        cp_async16(smem_u32(vd), src + v_off);
      } else {
        *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

  const int first_base = k0 + warp * 16;
  const int stride = 64;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (first_base + s * stride < k1) load_tile(first_base + s * stride, s);
    cp_async_commit();
  }
  int n_iter = 0;
  for (int base = first_base; base < k1; base += stride, ++n_iter) {
    const int ahead = base + (STAGES - 1) * stride;
    if (ahead < k1) load_tile(ahead, (n_iter + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncwarp();
    const bf16* kt = my_stages + (n_iter % STAGES) * STAGE_ELEMS;
    const bf16* vt = kt + 16 * LDS;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b[4];
      const int row = (lane >> 4) * 8 + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(b, smem_u32(kt + row * LDS + col));
      mma_bf16(s[0], qf[kk], b[0], b[1]);
      mma_bf16(s[1], qf[kk], b[2], b[3]);
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = base + n * 8 + 2 * (lane & 3) + (e & 1);
        s[n][e] = key < k1 ? s[n][e] * scale_log2 : -INFINITY;
      }
      mx_lo = fmaxf(mx_lo, fmaxf(s[n][0], s[n][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[n][2], s[n][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);   // finite: key `base` is always valid
    const float c_lo = exp2f(m_lo - mn_lo), c_hi = exp2f(m_hi - mn_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    l_lo *= c_lo;
    l_hi *= c_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= c_lo;
      o[i][1] *= c_lo;
      o[i][2] *= c_hi;
      o[i][3] *= c_hi;
    }
    uint32_t pa[4];
    {
      const float e0 = exp2f(s[0][0] - mn_lo), e1 = exp2f(s[0][1] - mn_lo);
      const float e2 = exp2f(s[0][2] - mn_hi), e3 = exp2f(s[0][3] - mn_hi);
      const float f0 = exp2f(s[1][0] - mn_lo), f1 = exp2f(s[1][1] - mn_lo);
      const float f2 = exp2f(s[1][2] - mn_hi), f3 = exp2f(s[1][3] - mn_hi);
      l_lo += e0 + e1 + f0 + f1;
      l_hi += e2 + e3 + f2 + f3;
      pa[0] = pack_bf16(e0, e1);
      pa[1] = pack_bf16(e2, e3);
      pa[2] = pack_bf16(f0, f1);
      pa[3] = pack_bf16(f2, f3);
    }
#pragma unroll
    for (int d2 = 0; d2 < D / 16; ++d2) {
      uint32_t b[4];
      const int row = ((lane >> 3) & 1) * 8 + (lane & 7), col = d2 * 16 + (lane >> 4) * 8;
      ldmatrix_x4_trans(b, smem_u32(vt + row * LDS + col));
      mma_bf16(o[2 * d2], pa, b[0], b[1]);
      mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // ---- merge the four warps in shared memory (the staging buffers are free now)
  __syncthreads();
  float* c_o = reinterpret_cast<float*>(stage_base);          // [4][16][D]
  float* c_m = c_o + 4 * 16 * D;                              // [4][16]
  float* c_l = c_m + 4 * 16;                                  // [4][16]
  {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int col = n * 8 + 2 * (lane & 3);
      c_o[(warp * 16 + r_lo) * D + col] = o[n][0];
      c_o[(warp * 16 + r_lo) * D + col + 1] = o[n][1];
      c_o[(warp * 16 + r_hi) * D + col] = o[n][2];
      c_o[(warp * 16 + r_hi) * D + col + 1] = o[n][3];
    }
    if ((lane & 3) == 0) {
      c_m[warp * 16 + r_lo] = m_lo;
      c_m[warp * 16 + r_hi] = m_hi;
      c_l[warp * 16 + r_lo] = l_lo;
      c_l[warp * 16 + r_hi] = l_hi;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += 128) {
    const int row = idx / D, dim = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, c_m[w * 16 + row]);
    float O = 0.0f, L = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(c_m[w * 16 + row] - M);
        O += f * c_o[(w * 16 + row) * D + dim];
        L += f * c_l[w * 16 + row];
      }
    }
    const int head = g * G + row;
    if (num_splits == 1) {
      out[((size_t)t * nq + head) * D + dim] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    } else {
      fin_o[row * D + dim] = O;
      if (dim == 0) {
        fin_m[row] = M;
        fin_l[row] = L;
      }
    }
  }
  if (num_splits == 1) return;
  // ---- merge over the cluster: block `split` takes dims [split * D / n, (split + 1) * D / n) of every
  //      head and reads all blocks' (maximum, sum, output) through distributed shared memory, in block order
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  const int DS = D / num_splits;
  for (int idx = tid; idx < G * DS; idx += 128) {
    const int row = idx / DS, dim = split * DS + idx % DS;
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      if (c < num_splits) {
        ms[c] = cluster.map_shared_rank(fin_m, c)[row];
        ls[c] = cluster.map_shared_rank(fin_l, c)[row];
        os[c] = cluster.map_shared_rank(fin_o, c)[row * D + dim];
      } else {
        ms[c] = -INFINITY;
        ls[c] = os[c] = 0.0f;
      }
    }
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) M = fmaxf(M, ms[c]);
    float O = 0.0f, L = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float f = exp2f(ms[c] - M);
        O += f * os[c];
        L += f * ls[c];
      }
    }
    out[((size_t)t * nq + g * G + row) * D + dim] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
  }
  cluster.sync();                                       // nobody leaves while its shared memory is being read
}

// ------------------------------------------- decoded tokens, pages fetched by TMA
// The same work as attn_decode_kernel for page sizes that are multiples of 16 and
// head sizes that are multiples of 64: a 16-key tile lies inside one page, so each
// warp's lane 0 fetches it with cp.async.bulk.tensor boxes [16 keys x 64 elements]
// (128-byte swizzle) from the pool seen as a matrix [pages * 2 * nkv * page_size, D],
// and the warp waits on the stage's mbarrier.  No per-lane address arithmetic, no
// padding: ldmatrix reads the swizzled tiles without bank conflicts.  Keys of a tile
// beyond the token's range get zero weight; what the page holds there is finite (the
// pool starts as zeros and only finite values are ever written to it).
template <int D, int STAGES, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap pool_map, const bf16* __restrict__ q,
                       const int* __restrict__ block_table, const int4* __restrict__ decode_meta,
                       bf16* __restrict__ out, int nq, int nkv, int page_size, int page_shift, int max_blocks,
                       int num_pages, int window, float scale_log2, int tbl_cap, int* __restrict__ error_flag) {
  constexpr int LDS = D + 8;
  constexpr int CPR = D / 8;
  constexpr int HALVES = D / 64;
  constexpr int TILE_BYTES = 16 * D * 2;                // one K or V tile: HALVES boxes of 2 KB
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int STAGE_BYTES_ALL = WARPS * STAGES * STAGE_BYTES;
  constexpr int THREADS = WARPS * 32;
  constexpr int MERGE_BYTES = (WARPS * 16 * D + 2 * WARPS * 16) * 4;
  constexpr int FIN_BYTES = (16 * D + 32) * 4;
  constexpr int WORK_BYTES = STAGE_BYTES_ALL > MERGE_BYTES + FIN_BYTES ? STAGE_BYTES_ALL : MERGE_BYTES + FIN_BYTES;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* stage_base =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  float* fin_o = reinterpret_cast<float*>(stage_base + MERGE_BYTES);     // [16][D], behind the warps' merge buffers
  float* fin_m = fin_o + 16 * D;
  float* fin_l = fin_m + 16;
  bf16* q_s = reinterpret_cast<bf16*>(stage_base + WORK_BYTES);           // [16][LDS]
  uint64_t* bars = reinterpret_cast<uint64_t*>(q_s + 16 * LDS);          // [warps][STAGES]
  int* tbl_s = reinterpret_cast<int*>(bars + WARPS * STAGES);                // [tbl_cap]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int item = blockIdx.x, g = blockIdx.y, split = blockIdx.z, num_splits = gridDim.z;
  const int G = nq / nkv;
  if (tid == 0) {
    for (int i = 0; i < WARPS * STAGES; ++i) mbar_init(smem_addr(bars + i), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The step's metadata, the block table and every key but the token's own were written before this
  // step's kernels began: tables are copied and the first tiles are on their way before the kernel in
  // front (which writes the token's own key and value, and the queries) is known to have finished.
  const int4 meta = decode_meta[item];
  const int t = meta.x;
  const int pos = meta.y;
  const int* table_g = block_table + (size_t)meta.z * max_blocks;
  const int* table = table_g;
  int blk_base = 0;

  const int kfirst = window > 0 ? max(0, pos - window + 1) : 0;
  const int kstart = kfirst & ~15;                      // tiles start on multiples of 16 so that one lies in one page
  const int kend = pos + 1;
  const int per_split = (((kend - kstart + num_splits - 1) / num_splits) + WARPS * 16 - 1) / (WARPS * 16) * (WARPS * 16);
  const int k0 = kstart + split * per_split;
  const int k1 = min(kend, k0 + per_split);
  if (k0 < k1) {
    const int b0 = k0 >> page_shift, b1 = (k1 - 1) >> page_shift;
    if (b1 - b0 + 1 <= tbl_cap) {
      for (int i = tid; i <= b1 - b0; i += THREADS) tbl_s[i] = table_g[b0 + i];
      table = tbl_s;
      blk_base = b0;
    }
  }
  __syncthreads();                                      // barriers initialised, table copied

  const uint32_t my_stage0 = smem_addr(stage_base) + warp * STAGES * STAGE_BYTES;
  const uint32_t my_bar0 = smem_addr(bars + warp * STAGES);
  auto issue_tile = [&](int base, int stage) {           // lane 0 only: keys base .. base + 15
    int page = table[(base >> page_shift) - blk_base];
    if (page < 0 || page >= num_pages) page = 0;
    const int off = base & (page_size - 1);
    const int yk = ((page * 2) * nkv + g) * page_size + off;
    const int yv = ((page * 2 + 1) * nkv + g) * page_size + off;
    const uint32_t dst = my_stage0 + stage * STAGE_BYTES, bar = my_bar0 + 8 * stage;
    mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
    for (int h = 0; h < HALVES; ++h) {
      tma_load_2d(dst + h * 2048, &pool_map, h * 64, yk, bar);
      tma_load_2d(dst + TILE_BYTES + h * 2048, &pool_map, h * 64, yv, bar);
    }
  };
  // byte offset of the 16-byte chunk holding elements [col, col + 8) of row `row` in a swizzled tile
  auto tile_off = [](int row, int col) -> uint32_t {
    return (uint32_t)((col >> 6) * 2048 + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4));
  };

  const int first_base = k0 + warp * 16;
  const int stride = WARPS * 16;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      const int base = first_base + s * stride;
      if (base < k1 && base + 16 <= pos) issue_tile(base, s);       // the tile with the token's own key waits
    }
  }
  pdl_wait();
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      const int base = first_base + s * stride;
      if (base < k1 && base + 16 > pos) issue_tile(base, s);
    }
  }
  for (int i = tid; i < 16 * CPR; i += THREADS) {
    const int row = i / CPR, c = i % CPR;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < G) v = *reinterpret_cast<const uint4*>(q + ((size_t)t * nq + g * G + row) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + row * LDS + c * 8) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8, col = kk * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[kk], smem_u32(q_s + row * LDS + col));
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;

  int n_iter = 0;
  bool ok = true;
  for (int base = first_base; base < k1; base += stride, ++n_iter) {
    const int stage = n_iter % STAGES;
    const int ahead = base + (STAGES - 1) * stride;
    if (lane == 0 && ahead < k1) {
      fence_proxy_async_smem();                           // the stage's last readers (ldmatrix) come before the copy
      issue_tile(ahead, (n_iter + STAGES - 1) % STAGES);
    }
    ok = mbar_wait(my_bar0 + 8 * stage, (n_iter / STAGES) & 1);
    if (!ok) break;
    const uint32_t kt = my_stage0 + stage * STAGE_BYTES, vt = kt + TILE_BYTES;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b[4];
      const int row = (lane >> 4) * 8 + (lane & 7), col = kk * 16 + ((lane >> 3) & 1) * 8;
      ldmatrix_x4(b, kt + tile_off(row, col));
      mma_bf16(s[0], qf[kk], b[0], b[1]);
      mma_bf16(s[1], qf[kk], b[2], b[3]);
    }
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = base + n * 8 + 2 * (lane & 3) + (e & 1);
        s[n][e] = (key < k1 && key >= kfirst) ? s[n][e] * scale_log2 : -INFINITY;
      }
      mx_lo = fmaxf(mx_lo, fmaxf(s[n][0], s[n][1]));
      mx_hi = fmaxf(mx_hi, fmaxf(s[n][2], s[n][3]));
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
    // a tile in front of the window's first key may hold no valid key at all
    const float mu_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, mu_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
    const float c_lo = exp2f(m_lo - mu_lo), c_hi = exp2f(m_hi - mu_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    l_lo *= c_lo;
    l_hi *= c_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= c_lo;
      o[i][1] *= c_lo;
      o[i][2] *= c_hi;
      o[i][3] *= c_hi;
    }
    uint32_t pa[4];
    {
      const float e0 = exp2f(s[0][0] - mu_lo), e1 = exp2f(s[0][1] - mu_lo);
      const float e2 = exp2f(s[0][2] - mu_hi), e3 = exp2f(s[0][3] - mu_hi);
      const float f0 = exp2f(s[1][0] - mu_lo), f1 = exp2f(s[1][1] - mu_lo);
      const float f2 = exp2f(s[1][2] - mu_hi), f3 = exp2f(s[1][3] - mu_hi);
      l_lo += e0 + e1 + f0 + f1;
      l_hi += e2 + e3 + f2 + f3;
      pa[0] = pack_bf16(e0, e1);
      pa[1] = pack_bf16(e2, e3);
      pa[2] = pack_bf16(f0, f1);
      pa[3] = pack_bf16(f2, f3);
    }
#pragma unroll
    for (int d2 = 0; d2 < D / 16; ++d2) {
      uint32_t b[4];
      const int row = ((lane >> 3) & 1) * 8 + (lane & 7), col = d2 * 16 + (lane >> 4) * 8;
      ldmatrix_x4_trans(b, vt + tile_off(row, col));
      mma_bf16(o[2 * d2], pa, b[0], b[1]);
      mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
    }
    __syncwarp();
  }
  pdl_launch_dependents();                 // the keys are read: the output projection may fetch its weights now
  if (!ok) {
    if (lane == 0) atomicExch(error_flag, 4);
    // copies that were issued and not waited for must land before the block leaves
    for (int n = n_iter + 1; n < n_iter + STAGES; ++n)
      if (first_base + n * stride < k1) mbar_wait(my_bar0 + 8 * (n % STAGES), (n / STAGES) & 1);
  }
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  // ---- merge the four warps in shared memory (the staging buffers are free now)
  __syncthreads();
  float* c_o = reinterpret_cast<float*>(stage_base);          // [4][16][D]
  float* c_m = c_o + WARPS * 16 * D;
  float* c_l = c_m + WARPS * 16;
  {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int col = n * 8 + 2 * (lane & 3);
      c_o[(warp * 16 + r_lo) * D + col] = o[n][0];
      c_o[(warp * 16 + r_lo) * D + col + 1] = o[n][1];
      c_o[(warp * 16 + r_hi) * D + col] = o[n][2];
      c_o[(warp * 16 + r_hi) * D + col + 1] = o[n][3];
    }
    if ((lane & 3) == 0) {
      c_m[warp * 16 + r_lo] = m_lo;
      c_m[warp * 16 + r_hi] = m_hi;
      c_l[warp * 16 + r_lo] = l_lo;
      c_l[warp * 16 + r_hi] = l_hi;
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += THREADS) {
    const int row = idx / D, dim = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, c_m[w * 16 + row]);
    float O = 0.0f, L = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float f = exp2f(c_m[w * 16 + row] - M);
        O += f * c_o[(w * 16 + row) * D + dim];
        L += f * c_l[w * 16 + row];
      }
    }
    if (num_splits == 1) {
      out[((size_t)t * nq + g * G + row) * D + dim] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    } else {
      fin_o[row * D + dim] = O;
      if (dim == 0) {
        fin_m[row] = M;
        fin_l[row] = L;
      }
    }
  }
  if (num_splits == 1) return;
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  const int DS = D / num_splits;
  for (int idx = tid; idx < G * DS; idx += THREADS) {
    const int row = idx / DS, dim = split * DS + idx % DS;
    float ms[16], ls[16], os[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      if (c < num_splits) {
        ms[c] = cluster.map_shared_rank(fin_m, c)[row];
        ls[c] = cluster.map_shared_rank(fin_l, c)[row];
        os[c] = cluster.map_shared_rank(fin_o, c)[row * D + dim];
      } else {
        ms[c] = -INFINITY;
        ls[c] = os[c] = 0.0f;
      }
    }
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < 16; ++c) M = fmaxf(M, ms[c]);
    float O = 0.0f, L = 0.0f;
    if (M != -INFINITY) {
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float f = exp2f(ms[c] - M);
        O += f * os[c];
        L += f * ls[c];
      }
    }
    out[((size_t)t * nq + g * G + row) * D + dim] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
  }
  cluster.sync();
}

template <int D, int STAGES, int WARPS>
int launch_decode_tma_stages(const CUtensorMap& pool_map, const bf16* q, const int* block_table, const int4* decode_meta,
                             bf16* out, int num_items, int nq, int nkv, int page_size, int page_shift, int max_blocks,
                             int num_pages, int window, float scale_log2, int num_splits, int max_keys, int* error_flag,
                             cudaStream_t stream) {
  constexpr int stage_bytes = WARPS * STAGES * 2 * 16 * D * 2;
  constexpr int merge_bytes = (WARPS * 16 * D + 2 * WARPS * 16) * 4;
  constexpr int fin_bytes = (16 * D + 32) * 4;
  constexpr int work_bytes = stage_bytes > merge_bytes + fin_bytes ? stage_bytes : merge_bytes + fin_bytes;
  constexpr int keys_round = WARPS * 16;
  const int per_split = (((max_keys + 16 + num_splits - 1) / num_splits) + keys_round - 1) / keys_round * keys_round;
  int tbl_cap = per_split / page_size + 2;
  if (tbl_cap > 8192) tbl_cap = 0;
  const int smem = 1024 + work_bytes + 16 * (D + 8) * 2 + WARPS * STAGES * 8 + tbl_cap * 4;
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, STAGES, WARPS>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  if (num_splits > 8) {                                   // a cluster of 16 is beyond the portable size
    static bool allowed = false;
    if (!allowed) {
      cudaError_t e = cudaFuncSetAttribute(attn_decode_tma_kernel<D, STAGES, WARPS>,
                                           cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) return (int)e;
      allowed = true;
    }
  }
  return launch_pdl(attn_decode_tma_kernel<D, STAGES, WARPS>, dim3(num_items, nkv, num_splits), dim3(WARPS * 32),
                    (size_t)smem, stream, num_splits, pool_map, q, block_table, decode_meta, out, nq, nkv, page_size,
                    page_shift, max_blocks, num_pages, window, scale_log2, tbl_cap, error_flag);
}

// Four warps with three 16-key tiles in flight each (96 KB a block at head size 128) feed the HBM when two blocks
// sit on every SM.  A grid that leaves a third of the SMs empty (one to three decoded tokens) is bound by the pace
// of a warp's tile loop and by what a block has in flight: it runs with eight warps a block (a decode step of the
// 7B shape at batch 1, 64 blocks: 2.75 -> 2.68 ms at 4,096 keys, 3.39 -> 3.07 ms at 32,768; batch 3, 96 blocks:
// 2.89 -> 2.80 and 4.20 -> 3.53 ms).  From 128 blocks on the larger blocks no longer all find room at once
// (batch 2 with clusters of 16 at 32,768 keys: 3.46 -> 3.68 ms; batch 4: 4.25 -> 4.55 ms).
template <int D>
int launch_decode_tma(const CUtensorMap& pool_map, const bf16* q, const int* block_table, const int4* decode_meta,
                      bf16* out, int num_items, int nq, int nkv, int page_size, int page_shift, int max_blocks,
                      int num_pages, int window, float scale_log2, int num_splits, int max_keys, int* error_flag,
                      cudaStream_t stream) {
  constexpr int STAGES = D <= 128 ? 3 : 2;
  const long long blocks = (long long)num_items * nkv * num_splits;
  const int keys_per_block = max_keys / (num_splits > 0 ? num_splits : 1);
#define ARGS pool_map, q, block_table, decode_meta, out, num_items, nq, nkv, page_size, page_shift, max_blocks, num_pages, \
             window, scale_log2, num_splits, max_keys, error_flag, stream
  if (D <= 128 && blocks <= 104 && keys_per_block >= 8 * 16) return launch_decode_tma_stages<D, STAGES, 8>(ARGS);
  return launch_decode_tma_stages<D, STAGES, 4>(ARGS);
#undef ARGS
}

template <int D>
int launch_prefill(const bf16* q, const bf16* kv_pool, const int* block_table, const int* tiles, const int* req_slot,
                   bf16* out, int num_tiles, int nq, int nkv, int page_size, int page_shift, int max_blocks,
                   int num_pages, int window, float scale_log2, int max_keys, cudaStream_t stream) {
  constexpr int KT = 64;                                // keys per tile
  constexpr int tile_bytes = (64 + 4 * KT) * (D + 8) * 2;
  int tbl_cap = max_keys / page_size + 2;               // entries a tile can need
  if (tbl_cap > 8192) tbl_cap = 0;                      // too long to copy: look pages up in global memory
  const int smem = tile_bytes + tbl_cap * 4;
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<D, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  dim3 grid(num_tiles * 4, nq);
  attn_prefill_kernel<D, KT><<<grid, 128, smem, stream>>>(q, kv_pool, block_table, tiles, req_slot, out, nq, nkv, page_size,
                                                      page_shift, max_blocks, num_pages, window, scale_log2, tbl_cap);
  IFX_CHECK_LAUNCH();
  return 0;
}

template <int D>
int launch_decode(const bf16* q, const bf16* kv_pool, const int* block_table, const int4* decode_meta, bf16* out,
                  int num_items, int nq, int nkv, int page_size, int page_shift, int max_blocks, int num_pages,
                  int window, float scale_log2, int num_splits, int max_keys, cudaStream_t stream) {
  constexpr int STAGES = D <= 128 ? 3 : 2;
  constexpr int stage_bytes = 4 * STAGES * 2 * 16 * (D + 8) * 2;
  constexpr int merge_bytes = (4 * 16 * D + 2 * 4 * 16) * 4;
  const int per_split = (((max_keys + num_splits - 1) / num_splits) + 63) / 64 * 64;
  int tbl_cap = per_split / page_size + 2;              // entries a split can need
  if (tbl_cap > 8192) tbl_cap = 0;
  constexpr int fin_bytes = (16 * D + 32) * 4;
  constexpr int work_bytes = stage_bytes > merge_bytes + fin_bytes ? stage_bytes : merge_bytes + fin_bytes;
  const int smem = 16 * (D + 8) * 2 + work_bytes + tbl_cap * 4;
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_items, nkv, num_splits);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = num_splits;
  cfg.attrs = attr;
  cfg.numAttrs = num_splits > 1 ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attn_decode_kernel<D, STAGES>, q, kv_pool, block_table, decode_meta, out, nq,
                                     nkv, page_size, page_shift, max_blocks, num_pages, window, scale_log2, tbl_cap);
  if (e != cudaSuccess) return (int)e;
  return 0;
}

static int shift_of(int page_size) {
  if (page_size <= 0 || (page_size & (page_size - 1))) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

}  // namespace ifx

using namespace ifx;

#define IFX_DISPATCH_D(d, CALL)                    \
  switch (d) {                                     \
    case 16: return CALL(16);                      \
    case 32: return CALL(32);                      \
    case 48: return CALL(48);                      \
    case 64: return CALL(64);                      \
    case 80: return CALL(80);                      \
    case 96: return CALL(96);                      \
    case 112: return CALL(112);                    \
    case 128: return CALL(128);                    \
    case 256: return CALL(256);                    \
    default: return IFX_E_BADARG;                  \
  }

extern "C" {

// 1 if the tiled kernels take this head size, else 0.
int ifx_attention_mma_supports(int d) {
  return d == 16 || d == 32 || d == 48 || d == 64 || d == 80 || d == 96 || d == 112 || d == 128 || d == 256;
}

// tiles: int32 [num_tiles, 4] = (request index, first flat row, rows <= 256, first position).
// max_keys: no request of the step holds more keys than this (sizes the shared-memory copy of the block table).
int ifx_attention_prefill_bf16(const void* q, const void* kv_pool, const int* block_table, const int* tiles,
                               const int* req_slot, void* out, int num_tiles, int nq, int nkv, int d, int page_size,
                               int max_blocks, int num_pages, int window, float scale, int max_keys, int* error_flag,
                               cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || page_size <= 0 || max_blocks <= 0 || nq > 65535 || !(scale > 0.0f))
    return IFX_E_BADARG;                                  // the kernels take the maximum before scaling
  const float scale_log2 = scale * 1.4426950408889634f;
  const int ps = shift_of(page_size);
#define CALL(DD)                                                                                                   \
  launch_prefill<DD>((const bf16*)q, (const bf16*)kv_pool, block_table, tiles, req_slot, (bf16*)out, num_tiles, nq, \
                     nkv, page_size, ps, max_blocks, num_pages, window, scale_log2, max_keys, stream)
  IFX_DISPATCH_D(d, CALL)
#undef CALL
}

// The largest cluster (blocks that share one token's keys) the decode kernel takes for this head and page size.
int ifx_attention_decode_max_splits(int d, int page_size) {
  const int ps = shift_of(page_size);
  return (ps >= 4 && (d == 64 || d == 128)) ? 16 : 8;
}

// decode_meta: int32 [num_items, 4] = (flat token row, position, request slot, unused).
// error_flag: device int that the TMA variant sets if a bounded wait runs out (nullptr: cp.async variant only).
// num_splits: 1, 2, 4 or 8 blocks (one cluster) share a token's key range; it must divide d.  16 where
// ifx_attention_decode_max_splits says so (the TMA variant, a cluster size beyond the portable 8).
// max_keys: no token of the step sees more keys than this.
int ifx_attention_decode_bf16(const void* q, const void* kv_pool, const int* block_table, const int* decode_meta,
                              void* out, int num_items, int nq, int nkv, int d, int page_size, int max_blocks,
                              int num_pages, int window, float scale, int num_splits, int max_keys, int* error_flag,
                              cudaStream_t stream) {
  if (num_items <= 0) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv || nq / nkv > 16 || page_size <= 0 || max_blocks <= 0 || nkv > 65535 ||
      nq > 65535)
    return IFX_E_BADARG;
  const int ps = shift_of(page_size);
  const bool tma = ps >= 4 && d % 64 == 0 && error_flag != nullptr;
  if (!(num_splits == 1 || num_splits == 2 || num_splits == 4 || num_splits == 8 || (num_splits == 16 && tma)) ||
      d % num_splits)
    return IFX_E_BADARG;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (tma) {                                                    // pages of 16, 32, ... tokens: the TMA kernel
    CUtensorMap pool_map;
    const long long rows = (long long)num_pages * 2 * nkv * page_size;
    int rc = pool_tensor_map(&pool_map, kv_pool, rows, d);
    if (rc) return rc;
#define CALL_TMA(DD)                                                                                              \
  return launch_decode_tma<DD>(pool_map, (const bf16*)q, block_table, (const int4*)decode_meta, (bf16*)out,       \
                               num_items, nq, nkv, page_size, ps, max_blocks, num_pages, window, scale_log2,      \
                               num_splits, max_keys, error_flag, stream)
    if (d == 64) CALL_TMA(64);
    if (d == 128) CALL_TMA(128);
    if (d == 256) CALL_TMA(256);
#undef CALL_TMA
  }
#define CALL(DD)                                                                                                  \
  launch_decode<DD>((const bf16*)q, (const bf16*)kv_pool, block_table, (const int4*)decode_meta, (bf16*)out,     \
                    num_items, nq, nkv, page_size, ps, max_blocks, num_pages, window, scale_log2, num_splits,     \
                    max_keys, stream)
  IFX_DISPATCH_D(d, CALL)
#undef CALL
}

}  // extern "C"
