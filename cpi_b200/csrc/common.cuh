// Shared helpers of the sm_100a kernel library: dtypes, conversions, reductions, error reporting.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a CUDA stream, launches
// asynchronously on that stream and returns 0, or a non-zero code after storing a message that
// cpi_last_error() returns.  Nothing here allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <utility>

namespace cpi {

enum DType : int { kF32 = 0, kBF16 = 1 };

void set_error(const char* fmt, ...);
void count_launch();                 // every kernel launch of the library is counted (cpi_launch_count)
int check_launch(const char* what);
int sm_count();                      // multiprocessors of the current device (1 when no device answers)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// load element i of a buffer whose dtype is only known at run time (small vectors: norm weights)
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
  return dtype == kF32 ? reinterpret_cast<const float*>(p)[i]
                       : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
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

// Block-wide sum in a fixed order; `scratch` holds >= 32 floats; every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < nw; ++i) r += scratch[i];
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int i = 1; i < nw; ++i) r = fmaxf(r, scratch[i]);
  return r;
}

// Programmatic dependent launch: a kernel launched with launch_pdl may start while the kernel before it
// in the stream is still running.  Every such kernel calls pdl_launch_dependents() early (so that its
// own successor may be scheduled) and pdl_wait() before it first reads or writes global memory that
// another kernel of the stream produces or reads; pdl_wait() returns once the preceding kernel has
// finished and its writes are visible.  What precedes the wait (barrier set-up, tensor-memory
// allocation, loads of weights, which no kernel writes) overlaps the predecessor's tail.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
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
  count_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace cpi

#define CPI_REQUIRE(cond, ...)                    \
  do {                                            \
    if (!(cond)) {                                \
      cpi::set_error(__VA_ARGS__);                \
      return 1;                                   \
    }                                             \
  } while (0)

// Calls `expr` with T bound to the C++ type of `dtype`.
#define CPI_DISPATCH_DTYPE(dtype, T, ...)                           \
  do {                                                              \
    if ((dtype) == cpi::kF32) { using T = float; __VA_ARGS__; }     \
    else if ((dtype) == cpi::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { cpi::set_error("unknown dtype code %d", (int)(dtype)); return 1; } \
  } while (0)
