// Shared helpers of the sm_100a kernels: element types, conversions, warp
// reductions with a fixed order, the paged-cache address rule and the error
// convention of the extern "C" launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
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
#if !defined(LLMX_TIMELINE)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define LLMX_MARK(id)
#else
// Built with -DLLMX_TIMELINE, the first thread of every kernel's first CTA records when it reached its
// dependency wait and when the wait returned (the global nanosecond timer), with the source line of the
// wait as the kernel's name.  Successive return times are the critical path of a chain of dependent
// kernels, measured in place (inside a replayed graph, with programmatic launch overlap), which no
// serialising profiler shows.  Every library keeps its own records; llmx_timeline_read() copies them out
// and starts over.  Off by default: the records cost a few instructions and an atomic per kernel.
#define LLMX_TIMELINE_MAX 65536
static __device__ unsigned long long llmx_timeline_records[3 * LLMX_TIMELINE_MAX];
static __device__ unsigned int llmx_timeline_count;
__device__ __forceinline__ unsigned long long llmx_global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void pdl_wait_at(int line) {
  const bool rec = (threadIdx.x | threadIdx.y | threadIdx.z | blockIdx.x | blockIdx.y | blockIdx.z) == 0;
  unsigned long long t0 = 0;
  if (rec) t0 = llmx_global_ns();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (rec) {
    const unsigned long long t1 = llmx_global_ns();
    const unsigned int i = atomicAdd(&llmx_timeline_count, 1u);
    if (i < LLMX_TIMELINE_MAX) {
      llmx_timeline_records[3 * i] = (unsigned long long)line;
      llmx_timeline_records[3 * i + 1] = t0;
      llmx_timeline_records[3 * i + 2] = t1;
    }
  }
}
#define pdl_wait() pdl_wait_at(__LINE__)
// A mark inside a kernel, by whichever thread calls it: (1000000 + id, linear CTA index, time).
__device__ __forceinline__ void llmx_mark(int id) {
  const unsigned int i = atomicAdd(&llmx_timeline_count, 1u);
  if (i < LLMX_TIMELINE_MAX) {
    llmx_timeline_records[3 * i] = 1000000ull + (unsigned long long)id;
    llmx_timeline_records[3 * i + 1] = blockIdx.x + gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    llmx_timeline_records[3 * i + 2] = llmx_global_ns();
  }
}
#define LLMX_MARK(id) llmx_mark(id)
// out: room for 3 * max_records words (line, reached, returned).  Returns the number of records copied, or the
// negated cudaError_t of a failed call.
extern "C" __attribute__((visibility("default"))) int llmx_timeline_read(unsigned long long* out, int max_records) {
  unsigned int n = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&n, llmx_timeline_count, sizeof(n));
  if (e != cudaSuccess) return -(int)e;
  if (n > LLMX_TIMELINE_MAX) n = LLMX_TIMELINE_MAX;
  if ((int)n > max_records) n = (unsigned int)max_records;
  if (n) e = cudaMemcpyFromSymbol(out, llmx_timeline_records, (size_t)n * 3 * sizeof(unsigned long long));
  const unsigned int zero = 0;
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(llmx_timeline_count, &zero, sizeof(zero));
  return e == cudaSuccess ? (int)n : -(int)e;
}
#endif
// ---------------------------------------------------------------------------
// Failure reports.  A kernel whose bounded wait ran out (or that met something it cannot do) says so in one
// word per library, which lives in host memory that the device can write (llmx_set_status_word): the host
// reads it without a copy whenever it has waited for a step anyway.  The first report since the host last
// cleared the word stays.
// ---------------------------------------------------------------------------
static __device__ int* llmx_status_word;
__device__ __forceinline__ void llmx_report(int code) {
  volatile int* p = llmx_status_word;
  if (p && *p == 0) {
    *p = code;
    __threadfence_system();
  }
}
// host_word: one int of page-locked host memory (nullptr: reports stay in the library)
extern "C" __attribute__((visibility("default"))) int llmx_set_status_word(int* host_word) {
  void* dev_ptr = nullptr;
  if (host_word) {
    cudaError_t e = cudaHostGetDevicePointer(&dev_ptr, host_word, 0);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaMemcpyToSymbol(llmx_status_word, &dev_ptr, sizeof(dev_ptr));
}

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Whether a launch may overlap the kernel before it (programmatic stream serialization).  The host switches
// it per step with llmx_set_pdl(); LLMX_NO_PDL=1 in the environment switches it off for good (for telling a
// fault of a kernel from a fault of the overlap between two).
static int g_llmx_pdl_on = 1;
extern "C" __attribute__((visibility("default"))) void llmx_set_pdl(int on) { g_llmx_pdl_on = on ? 1 : 0; }
static inline int llmx_pdl_allowed() {
  static int off = -1;
  if (off < 0) {
    const char* e = getenv("LLMX_NO_PDL");
    off = (e && e[0] == '1') ? 1 : 0;
  }
  return off ? 0 : g_llmx_pdl_on;
}

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
  attr[0].val.programmaticStreamSerializationAllowed = llmx_pdl_allowed();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same for a grid whose CTAs form clusters of `cluster_x` along x (gridDim.x a multiple of it).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                             cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = llmx_pdl_allowed();
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

#ifdef __CUDACC__
// Makes this library's CUDA module resident on the current device without launching anything of its own
// work: the caller does this while the GPU is idle, so that no module is loaded in the middle of a step.
static __global__ void llmx_touch_kernel(int* p) {
  if (p) *p = 0;
}
extern "C" __attribute__((visibility("default"))) int llmx_touch() {
  cudaFuncAttributes a;
  cudaError_t e = cudaFuncGetAttributes(&a, llmx_touch_kernel);
  if (e != cudaSuccess) return (int)e;
  llmx_touch_kernel<<<1, 1>>>(nullptr);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaDeviceSynchronize();
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
