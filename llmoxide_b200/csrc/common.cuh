// Shared helpers of the sm_100a kernels: element types, conversions, warp
// reductions with a fixed order, the paged-cache address rule and the error
// convention of the extern "C" launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLMX_API extern "C" __attribute__((visibility("default")))

// Launchers return 0 or a negative code for a refused argument, or the
// positive cudaError_t of a failed launch.
#define LLMX_REFUSED(code) (-(code))
#define LLMX_LAUNCH_STATUS() ((int)cudaGetLastError())

typedef __nv_bfloat16 bf16;

// dtype tags passed through the C interface
enum { LLMX_F32 = 0, LLMX_BF16 = 1 };

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of this library is launched
// with the stream-serialization attribute and begins with
// pdl_launch_dependents() (the next kernel's CTAs may be scheduled as soon as
// all of this kernel's have started) and pdl_wait() (block until the kernel
// before has finished and its writes are visible) ahead of its first read or
// write of anything another kernel touches.  Decode steps are chains of short
// kernels; this overlaps each launch and prologue with the kernel before.
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// Tokens per cache page.  A sequence's position p lives in its logical page
// p / PAGE at row p % PAGE; the block table maps logical to physical pages.
#define LLMX_PAGE 64

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// Butterfly reductions: every lane ends with the same value, and the order of
// the additions is fixed by the lane numbers alone.
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

// Block-wide sum through shared memory, fixed order: warp butterflies, then
// the first warp adds the per-warp sums.  `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < n_warps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// Element offset of (physical page, kv head, row in page, dim 0) in one cache
// entry laid out [n_pages][G][PAGE][D].
__device__ __forceinline__ size_t cache_row_offset(int page, int g, int row, int G, int D) {
  return (((size_t)page * G + g) * LLMX_PAGE + row) * (size_t)D;
}
