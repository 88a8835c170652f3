// Row-wise kernels: token embedding, RMS norm, row gather, expert-output combine.
//
// Formulas (file:line of kurulav1/cpi):
//   embedding   x = Emb[token]                                   src/engine/llama4_cpu_engine.cpp:294-298
//   rmsnorm     y = x * rsqrt(mean(x^2) + eps) * w, fp32 sums    src/engine/llama4_cpu_engine.cpp:47-62,
//                                                                src/kernels/kernels.cu:36-99
// The residual stream is float32 in both precisions; norm outputs take the activation dtype.
#include "common.cuh"

namespace cpi {

template <typename TT>
__global__ void embedding_kernel(const int* __restrict__ tokens, const TT* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, int* __restrict__ err) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {              // never read out of range: flag it and write zeros
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.f;
    return;
  }
  const TT* row = table + (size_t)tok * hidden;
  float* dst = out + (size_t)t * hidden;
  if (sizeof(TT) == 2 && hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    // eight elements per thread and load: a row is only a few kilobytes, what counts is one round trip
    const uint4* r16 = reinterpret_cast<const uint4*>(row);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
      const uint4 raw = r16[i];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]), c = __bfloat1622float2(h2[2]), d = __bfloat1622float2(h2[3]);
      reinterpret_cast<float4*>(dst)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
      reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32(row[i]);
}

// One block per row.  The sum of squares is taken in a fixed order (thread-strided, then a warp
// tree, then warps in order), so a row's result does not depend on the other rows of the launch.
// Rows of up to 16 elements per thread stay in registers between the two passes.
template <typename TX, typename TO>
__global__ void rmsnorm_kernel(const TX* __restrict__ x, long x_stride, const int* __restrict__ rows,
                               const void* __restrict__ w, int w_dtype, TO* __restrict__ out,
                               long out_stride, int n, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const TX* xr = x + (size_t)(rows ? rows[r] : r) * x_stride;
  TO* o = out + (size_t)r * out_stride;
  constexpr int PER = 16;
  if (n <= PER * (int)blockDim.x) {
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      v[j] = i < n ? to_f32(xr[i]) : 0.f;
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n) {
        float y = v[j] * inv;
        if (w) y *= load_any(w, w_dtype, i);
        o[i] = from_f32<TO>(y);
      }
    }
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_f32(xr[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = to_f32(xr[i]) * inv;
    if (w) v *= load_any(w, w_dtype, i);
    o[i] = from_f32<TO>(v);
  }
}

// float32 rows whose length is a multiple of 4: 16-byte loads, the row kept in registers (up to 8192
// elements).  The norm weights are no kernel's output, so they are fetched (as vectors too) before the wait
// on the preceding kernel; after the reduction there is only arithmetic and one vector store per group.
template <typename TO>
__global__ void __launch_bounds__(256) rmsnorm_vec4_kernel(const float* __restrict__ x, long x_stride,
                                                           const int* __restrict__ rows, const void* __restrict__ w,
                                                           int w_dtype, TO* __restrict__ out, long out_stride, int n,
                                                           float eps) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  constexpr int PER = 8;
  const int r = blockIdx.x, n4 = n >> 2;
  float4 g[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 256;
    g[j] = make_float4(1.f, 1.f, 1.f, 1.f);
    if (w && i < n4) {
      if (w_dtype == kF32) {
        g[j] = reinterpret_cast<const float4*>(w)[i];
      } else {
        const uint2 raw = reinterpret_cast<const uint2*>(w)[i];
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        g[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
      }
    }
  }
  pdl_wait();
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * x_stride);
  float4 v[PER];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 256;
    v[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  TO* o = out + (size_t)r * out_stride;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < n4) {
      // (x * inv) * weight, in this order, as the scalar kernel does
      const float y0 = v[j].x * inv * g[j].x, y1 = v[j].y * inv * g[j].y, y2 = v[j].z * inv * g[j].z, y3 = v[j].w * inv * g[j].w;
      if (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + 4 * i) = make_float4(y0, y1, y2, y3);
      } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&a);
        pk.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(o) + 4 * i) = pk;
      }
    }
  }
}

// residual[t] += sum_k y[row_of_slot[t*K + k]] in the order k = 0..K-1.
template <typename TY>
__global__ void moe_combine_kernel(float* __restrict__ residual, const TY* __restrict__ y,
                                   const int* __restrict__ row_of_slot, int top_k, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < hidden; i += gridDim.y * blockDim.x) {
    float acc = residual[(size_t)t * hidden + i];
    for (int k = 0; k < top_k; ++k) {
      const int r = row_of_slot[t * top_k + k];
      acc += to_f32(y[(size_t)r * hidden + i]);
    }
    residual[(size_t)t * hidden + i] = acc;
  }
}

__device__ __forceinline__ float4 load4_f32(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4_f32(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// The same sum, four features per thread and one pass: every load of a thread is in flight at once
// (hidden a multiple of 4, all rows 16-byte aligned).  Same order of additions, so the same bits.
template <typename TY>
__global__ void moe_combine_vec4_kernel(float* __restrict__ residual, const TY* __restrict__ y,
                                        const int* __restrict__ row_of_slot, int top_k, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (i >= hidden) return;
  float* res = residual + (size_t)t * hidden + i;
  float4 acc = load4_f32(res);
  for (int k0 = 0; k0 < top_k; k0 += 4) {
    float4 v[4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      if (k0 + kk < top_k) v[kk] = load4_f32(y + (size_t)row_of_slot[t * top_k + k0 + kk] * hidden + i);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      if (k0 + kk < top_k) { acc.x += v[kk].x; acc.y += v[kk].y; acc.z += v[kk].z; acc.w += v[kk].w; }
  }
  *reinterpret_cast<float4*>(res) = acc;
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* g = gu + (size_t)t * 2 * inter;
  for (int i = threadIdx.x; i < inter; i += blockDim.x) {
    const float a = to_f32(g[i]), b = to_f32(g[inter + i]);
    out[(size_t)t * inter + i] = from_f32<T>(a / (1.0f + expf(-a)) * b);
  }
}

// dst[r, :] = src[rows[r], :]  (16-byte chunks; width * sizeof(T) must be a multiple of 16)
__global__ void gather_rows_kernel(const uint4* __restrict__ src, long src_stride16, const int* __restrict__ rows,
                                   uint4* __restrict__ dst, int chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const uint4* s = src + (size_t)rows[r] * src_stride16;
  uint4* d = dst + (size_t)r * chunks;
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) d[i] = s[i];
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_gather_rows(const void* src, long src_stride_bytes, const int* rows, void* dst, int n_rows,
                               int row_bytes, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(row_bytes % 16 == 0 && src_stride_bytes % 16 == 0, "gather_rows: rows of %d bytes (stride %ld) are not 16-byte multiples", row_bytes, src_stride_bytes);
  cpi::launch_pdl(gather_rows_kernel, n_rows, 128, 0, stream, (const uint4*)src, src_stride_bytes / 16, rows, (uint4*)dst, row_bytes / 16);
  return check_launch("gather_rows");
}

extern "C" int cpi_embedding(const int* tokens, const void* table, int table_dtype, float* out,
                             int n_tokens, int hidden, int vocab, int* err_flag, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embedding: bad sizes T=%d H=%d V=%d", n_tokens, hidden, vocab);
  CPI_DISPATCH_DTYPE(table_dtype, TT,
      cpi::launch_pdl(embedding_kernel<TT>, n_tokens, 256, 0, stream, tokens, (const TT*)table, out, hidden, vocab, err_flag));
  return check_launch("embedding");
}

extern "C" int cpi_rmsnorm(const void* x, int x_dtype, long x_stride, const int* rows, const void* w,
                           int w_dtype, void* out, int out_dtype, long out_stride, int n_rows, int n,
                           float eps, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(n_rows > 0 && n > 0, "rmsnorm: bad sizes rows=%d n=%d", n_rows, n);
  const int out_esz = out_dtype == kF32 ? 4 : 2;
  if (x_dtype == kF32 && n % 4 == 0 && n >= 1024 && n <= 8192 && x_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (out_stride * out_esz) % 16 == 0) {
    CPI_DISPATCH_DTYPE(out_dtype, TO,
        (cpi::launch_pdl(rmsnorm_vec4_kernel<TO>, n_rows, 256, 0, stream, (const float*)x, x_stride, rows, w, w_dtype,
                         (TO*)out, out_stride, n, eps)));
    return check_launch("rmsnorm");
  }
  const int threads = n <= 256 ? 64 : (n <= 2048 ? 256 : 512);
  CPI_DISPATCH_DTYPE(x_dtype, TX, CPI_DISPATCH_DTYPE(out_dtype, TO,
      (cpi::launch_pdl(rmsnorm_kernel<TX, TO>, n_rows, threads, 0, stream, (const TX*)x, x_stride, rows, w, w_dtype,
                                                              (TO*)out, out_stride, n, eps))));
  return check_launch("rmsnorm");
}

extern "C" int cpi_moe_combine(float* residual, const void* y, int y_dtype, const int* row_of_slot,
                               int n_tokens, int top_k, int hidden, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  const bool vec = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (y_dtype == kF32 || y_dtype == kBF16);
  if (vec) {
    const dim3 grid(n_tokens, (hidden / 4 + 127) / 128);
    if (y_dtype == kF32)
      cpi::launch_pdl(moe_combine_vec4_kernel<float>, grid, 128, 0, stream, residual, (const float*)y, row_of_slot, top_k, hidden);
    else
      cpi::launch_pdl(moe_combine_vec4_kernel<__nv_bfloat16>, grid, 128, 0, stream, residual, (const __nv_bfloat16*)y, row_of_slot, top_k, hidden);
    return check_launch("moe_combine");
  }
  CPI_DISPATCH_DTYPE(y_dtype, TY,
      cpi::launch_pdl(moe_combine_kernel<TY>, dim3(n_tokens, 1), 256, 0, stream, residual, (const TY*)y, row_of_slot, top_k, hidden));
  return check_launch("moe_combine");
}

extern "C" int cpi_swiglu(const void* gate_up, void* out, int dtype, int n_rows, int inter, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(swiglu_kernel<T>, n_rows, 256, 0, stream, (const T*)gate_up, (T*)out, inter));
  return check_launch("swiglu");
}
