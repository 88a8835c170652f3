// Kernels that run once, when a model is loaded: random weights, widening of half-precision tensors, and the
// transposition of the experts' matrices.
//
// The reference's counterpart is one conversion kernel, bfloat16 to float16, run over every weight at start-up
// (src/kernels/kernels_ops_matvec.cu:195-201, called from src/engine/llama4_cuda_engine_setup.cu:192-217); it has no
// random weights (its substitute is the .ll2c packing tool chain) and indexes the experts' matrices in their stored
// [in, out] layout.  Here weights stay bfloat16, float16 tensors are widened exactly to float32, the experts' matrices
// are turned once into [out, in], so that every contraction reads its weights along the reduction axis, and the
// random-weights mode draws each tensor with a counter-based generator whose bits do not depend on the device.
#include "common.cuh"
#include <cuda_fp16.h>

namespace cpi {

// Element i of a stream is a function of (stream seed, i) alone: SplitMix64's finaliser over i * golden ratio + seed,
// whose top 16 bits pick one of 65,536 values of the inverse normal distribution function (a float32 table made by
// the caller); the draw is that value times `std`, rounded to the output dtype.  The same integer arithmetic as the
// host-side generator (cpi_b200/weights/random_init.py): the same bits.
template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long start, long n, unsigned long long seed, float std,
                                     const float* __restrict__ table) {
  for (long k = (long)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += (long)gridDim.x * blockDim.x) {
    unsigned long long z = (unsigned long long)(start + k) * 0x9E3779B97F4A7C15ull + seed;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    out[k] = from_f32<T>(__ldg(table + (z >> 48)) * std);
  }
}

// float16 -> float32, exact.
__global__ void widen_f16_kernel(const __half* __restrict__ src, float* __restrict__ dst, long n) {
  for (long k = (long)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += (long)gridDim.x * blockDim.x)
    dst[k] = __half2float(src[k]);
}

// dst[g][c][r] = src[g][r][c] for matrices of `rows` x `cols`, through a 32 x 33 tile of shared memory so that reads
// and writes are both along rows.  grid (cols / 32, rows / 32, groups), block (32, 8).
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int cols) {
  __shared__ T tile[32][33];
  const size_t base = (size_t)blockIdx.z * rows * cols;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = src[base + (size_t)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[base + (size_t)c * rows + r] = tile[threadIdx.x][j];
  }
}

}  // namespace cpi

using namespace cpi;

// out[0 .. n) = draws start .. start + n - 1 of the stream `seed`, times std; `table`: 65,536 float32 on the device.
extern "C" int cpi_random_normal(void* out, int dtype, long start, long n, unsigned long long seed, float std,
                                 const float* table, cudaStream_t stream) {
  if (n <= 0) return 0;
  CPI_REQUIRE(table != nullptr, "random_normal: the table of the inverse normal distribution is missing");
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  count_launch();
  CPI_DISPATCH_DTYPE(dtype, T, (random_normal_kernel<T><<<blocks, 256, 0, stream>>>((T*)out, start, n, seed, std, table)));
  return check_launch("random_normal");
}

extern "C" int cpi_widen_f16(const void* src, float* dst, long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  count_launch();
  widen_f16_kernel<<<blocks, 256, 0, stream>>>((const __half*)src, dst, n);
  return check_launch("widen_f16");
}

// dst [groups, cols, rows] = src [groups, rows, cols] transposed in its last two axes; 2- or 4-byte elements.
extern "C" int cpi_transpose(const void* src, void* dst, int elem_bytes, long groups, int rows, int cols,
                             cudaStream_t stream) {
  if (groups <= 0 || rows <= 0 || cols <= 0) return 0;
  CPI_REQUIRE(elem_bytes == 2 || elem_bytes == 4, "transpose: elements of %d bytes (2 or 4)", elem_bytes);
  CPI_REQUIRE(groups <= 65535 && (rows + 31) / 32 <= 65535, "transpose: too many groups or rows (%ld, %d)", groups, rows);
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32, (unsigned)groups), block(32, 8);
  count_launch();
  if (elem_bytes == 2) transpose_kernel<unsigned short><<<grid, block, 0, stream>>>((const unsigned short*)src, (unsigned short*)dst, rows, cols);
  else transpose_kernel<unsigned int><<<grid, block, 0, stream>>>((const unsigned int*)src, (unsigned int*)dst, rows, cols);
  return check_launch("transpose");
}
