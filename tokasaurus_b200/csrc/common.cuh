// Shared helpers for the sm_100a kernels of this engine.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define TKB_EXPORT extern "C" __attribute__((visibility("default")))

// Bits of the device status word that kernels set instead of reading or writing out of range.
#define TKB_STATUS_BAD_TOKEN_ID 1
#define TKB_STATUS_BAD_PAGE 2
#define TKB_STATUS_WAIT_TIMEOUT 4

namespace tkb {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
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

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// A page id read from a block table, checked against the pool before it becomes an address: an id beyond the pool
// sets the status flag and is treated like -1 (the loaders then fill zeros; nothing is read out of range).
// Negative ids are legitimate: a page that was given back behind an attention window.  num_pages <= 0: the caller
// does not know the pool's size, nothing is checked.
__device__ __forceinline__ int checked_page(int page, int num_pages, int* status) {
  if (num_pages > 0 && page >= num_pages) {
    if (status != nullptr) atomicOr(status, TKB_STATUS_BAD_PAGE);
    return -1;
  }
  return page;
}
// The same for inner loops: no branch and no atomic there, the caller keeps `bad` in a register and reports it
// once, at its end, with report_bad_page().
__device__ __forceinline__ int checked_page(int page, int num_pages, bool& bad) {
  const bool b = num_pages > 0 && page >= num_pages;
  bad |= b;
  return b ? -1 : page;
}
__device__ __forceinline__ void report_bad_page(bool bad, int* status) {
  if (bad && status != nullptr) atomicOr(status, TKB_STATUS_BAD_PAGE);
}

// Programmatic dependent launch: a kernel launched with `launch_pdl` may start while the kernel
// before it in the stream is still running.  It must call grid_dependency_wait() before it reads
// anything an earlier kernel wrote and before it writes anything at all; what it does before that
// call (fetching weights, which no kernel writes) overlaps the earlier kernel.  Every kernel calls
// trigger_dependents() at its start so that its successor can be brought onto the SMs early; without a
// programmatic launch behind or before it, both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void trigger_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  return static_cast<int>(e);
}

// Number of SMs of the current device, asked once per process (the grids and work splits of the kernels are sized
// by it; no file holds the count of a particular GPU).  1 if the query fails: every split is then still right,
// only too coarse.
inline int sm_count() {
  static int cached = -1;
  if (cached < 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 1;
    cached = n;
  }
  return cached;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return static_cast<int>(e);
}

}  // namespace tkb
