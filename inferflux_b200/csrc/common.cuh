// Shared helpers of the sm_100a kernels: dtype conversion, warp/block reductions,
// argument checks.  Every exported function returns 0 on success, a positive
// cudaError_t, or a negative IFX_E_* code for arguments it refuses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IFX_DT_F32 0
#define IFX_DT_BF16 1

#define IFX_E_BADARG (-1)      // a size or option the kernel does not take
#define IFX_E_DTYPE (-2)       // unknown dtype code
#define IFX_E_ALIGN (-3)       // a pointer or stride that breaks an alignment rule
#define IFX_E_TOOBIG (-4)      // beyond a stated maximum

#define IFX_CHECK_LAUNCH()                         \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) return (int)e__;       \
  } while (0)

namespace ifx {

// Programmatic dependent launch: a kernel launched with launch_pdl may begin (set up
// its barriers, fetch weights) while the kernel before it in the stream is still
// draining; pdl_wait() returns once that kernel has completed and its writes are
// visible, and must come before the first access to anything it produced.  Every
// kernel launched this way calls pdl_wait() at some point, so completion stays
// transitive along the stream.  pdl_launch_dependents() lets the next kernel's
// blocks take the SM slots this kernel's blocks leave.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

extern int g_pdl_enabled;      // 1: launch_pdl sets the programmatic-serialization attribute
extern int g_shared_carveout;  // >= 0: percent of the SM's memory every launch_pdl kernel prefers as shared memory

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      int cluster_z, Args... args) {
  if (g_shared_carveout >= 0) {
    // Every kernel of the chain asks for the same split of the SM's memory into shared memory and L1, so that
    // no SM has to drain to change it between two kernels (measured: 3.30 -> 3.23 ms for a decode step of the
    // 7B shape at batch 8 with 100, 3.87 ms with 50).
    static const void* configured[64];                   // kernels of this signature seen so far
    static int num_configured = 0;
    const void* fn = reinterpret_cast<const void*>(kernel);
    bool seen = false;
    for (int i = 0; i < num_configured; ++i) seen = seen || configured[i] == fn;
    if (!seen) {
      cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, g_shared_carveout);
      if (num_configured < 64) configured[num_configured++] = fn;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z;
    ++n;
  }
  if (g_pdl_enabled) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return e == cudaSuccess ? 0 : (int)e;
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order
// of the additions depends only on the block size, so a row's result does not
// depend on which other rows are in the launch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                       // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

}  // namespace ifx
