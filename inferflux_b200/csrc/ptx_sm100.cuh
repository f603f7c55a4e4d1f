// PTX helpers shared by the kernels that use sm_100a's asynchronous machinery:
// mbarriers with bounded waits, TMA (cp.async.bulk.tensor) tile loads, and the host
// side of tensor maps.  No multicast form of any load is used anywhere.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <functional>
#include <mutex>
#include <unordered_map>

namespace ifx {

constexpr int kWaitLimit = 1 << 22;      // tries of a bounded mbarrier wait

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  False if it never came.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kWaitLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// The same with an L2 eviction policy (see l2_evict_first_policy).
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], "
      "[%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// Data that is read once (streamed weights) should leave L2 first, so that what is read again
// soon (activations, partial sums) stays.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Generic-proxy accesses to shared memory (ldmatrix, stores) that came before are ordered
// before asynchronous-proxy accesses (TMA writes) that come after.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
inline EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// A [rows, cols] row-major bfloat16 matrix, read in boxes of [box_rows, 64 elements] with the
// 128-byte swizzle.  Returns 0, -1 if the encoder is missing, -3 for a base or row pitch that
// is not 16-byte aligned, or 2000 + the driver's error.
inline int make_tensor_map_bf16(CUtensorMap* map, const void* base, long long rows, int cols, int box_rows) {
  EncodeTiledFn fn = tensor_map_encoder();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols % 8)) return -3;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

// Tensor maps of weight matrices ([rows, cols] bfloat16, boxes of [box_rows, 64]), made once per tensor and kept.
inline int weight_tensor_map(CUtensorMap* out, const void* base, long long rows, int cols, int box_rows) {
  struct Key {
    const void* base;
    long long rows;
    int cols, box;
    bool operator==(const Key& o) const { return base == o.base && rows == o.rows && cols == o.cols && box == o.box; }
  };
  struct Hash {
    size_t operator()(const Key& k) const {
      return std::hash<const void*>()(k.base) ^ (size_t)k.rows * 1000003u ^ (size_t)k.cols * 7919u ^ (size_t)k.box;
    }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  Key key{base, rows, cols, box_rows};
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

// Tensor maps of key/value pools (one per layer's pool, rows of one head's `d` elements, boxes of
// 16 rows), made once and kept.
inline int pool_tensor_map(CUtensorMap* out, const void* base, long long rows, int d) {
  struct Key {
    const void* base;
    long long rows;
    int d;
    bool operator==(const Key& o) const { return base == o.base && rows == o.rows && d == o.d; }
  };
  struct Hash {
    size_t operator()(const Key& k) const { return std::hash<const void*>()(k.base) ^ (size_t)k.rows * 31u ^ (size_t)k.d; }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> cache;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  Key key{base, rows, d};
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap m;
    int rc = make_tensor_map_bf16(&m, base, rows, d, 16);
    if (rc) return rc;
    it = cache.emplace(key, m).first;
  }
  *out = it->second;
  return 0;
}

}  // namespace ifx
