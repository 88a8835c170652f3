// Next-token choice on the device: greedy arg-max and temperature / top-k / top-p sampling.
//
// Reference semantics (file:line of kurulav1/cpi): temperature <= 0 takes the first maximum
// (src/engine/llama4_cuda_engine.cu:143-146; device arg-max src/kernels/kernels_ops_matvec.cu:421-454);
// otherwise logits / T, softmax over the whole vocabulary, keep the top_k most probable, walk them in
// descending order and stop once the kept mass reaches top_p (the token that crosses it is kept),
// renormalise, draw (src/engine/llama4_cuda_engine.cu:148-225).  Non-finite logits count as -inf and
// the rest are clamped to [-80, 80] first (:75-85).  The reference draws from an unseeded mt19937;
// here the uniform number comes from the caller, so a run is reproducible from its seed.
#include "common.cuh"

namespace cpi {

constexpr int SAMP_NT = 1024;

__device__ __forceinline__ float sanitize(float v) {
  if (!(fabsf(v) <= 3.0e38f)) return -INFINITY;       // NaN and +-inf
  return fminf(80.f, fmaxf(-80.f, v));
}

// (value, index) arg-max over the block, smallest index among equals; every thread gets the result.
__device__ void block_argmax(float& v, int& idx, float* sv, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { sv[warp] = v; si[warp] = idx; }
  __syncthreads();
  v = sv[0]; idx = si[0];
  for (int i = 1; i < nw; ++i)
    if (sv[i] > v || (sv[i] == v && si[i] < idx)) { v = sv[i]; idx = si[i]; }
}

__global__ void __launch_bounds__(SAMP_NT) argmax_kernel(const float* __restrict__ logits, long stride,
                                                         int vocab, int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (size_t)blockIdx.x * stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += SAMP_NT) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }               // strided scan keeps the smallest index per thread
  }
  block_argmax(best, bi, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// One block per row.  `work` is a float32 [rows, vocab] scratch the kernel overwrites.
__global__ void __launch_bounds__(SAMP_NT) sample_kernel(const float* __restrict__ logits, long stride,
                                                         float* __restrict__ work, int vocab,
                                                         const float* __restrict__ temperature,
                                                         const int* __restrict__ top_k,
                                                         const float* __restrict__ top_p,
                                                         const float* __restrict__ uniform,
                                                         int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float scratch[32];
  __shared__ float kept_p[256];
  __shared__ int kept_i[256];
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * stride;
  float* w = work + (size_t)r * vocab;
  const float T = temperature[r];
  if (!(T > 0.f)) {                                   // greedy
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMP_NT) {
      const float v = sanitize(row[i]);
      if (v > best) { best = v; bi = i; }
    }
    block_argmax(best, bi, sv, si);
    if (tid == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
    return;
  }
  const float inv_t = 1.0f / T;
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += SAMP_NT) {
    const float v = sanitize(row[i]) * inv_t;
    w[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, scratch);
  if (mx == -INFINITY) { if (tid == 0) out[r] = 0; return; }
  float sum = 0.f;
  for (int i = tid; i < vocab; i += SAMP_NT) {
    const float e = w[i] == -INFINITY ? 0.f : expf(w[i] - mx);
    w[i] = e;
    sum += e;
  }
  sum = block_sum(sum, scratch);
  const float inv_sum = 1.0f / sum;
  const int k = max(1, min(min(top_k[r], vocab), 256));
  const float tp = top_p[r];
  const bool use_p = tp > 0.f && tp < 1.f;
  float kept_sum = 0.f;
  int n_kept = 0;
  for (int j = 0; j < k; ++j) {                       // k rounds of arg-max with removal
    float best = -1.f; int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMP_NT) {
      const float v = w[i];
      if (v > best) { best = v; bi = i; }
    }
    block_argmax(best, bi, sv, si);
    if (!(best > 0.f)) break;
    if (tid == 0) { kept_p[n_kept] = best * inv_sum; kept_i[n_kept] = bi; w[bi] = -1.f; }
    kept_sum += best * inv_sum;
    ++n_kept;
    __syncthreads();
    if (use_p && kept_sum >= tp) break;
  }
  if (tid == 0) {
    if (n_kept == 0) { out[r] = 0; return; }
    float renorm = 0.f;
    for (int j = 0; j < n_kept; ++j) renorm += kept_p[j];
    const float u = uniform[r];
    float run = 0.f;
    int pick = kept_i[n_kept - 1];
    for (int j = 0; j < n_kept; ++j) {
      run += kept_p[j] / renorm;
      if (u <= run) { pick = kept_i[j]; break; }
    }
    out[r] = pick;
  }
}

// logits[r, id] /= penalty (if > 0) or *= penalty, once per distinct id of the row's history.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, long stride, int vocab,
                                          const int* __restrict__ ids, const int* __restrict__ id_offsets,
                                          const float* __restrict__ penalty) {
  const int r = blockIdx.x;
  const float pen = penalty[r];
  if (!(pen > 1.0f)) return;
  for (int j = id_offsets[r] + threadIdx.x; j < id_offsets[r + 1]; j += blockDim.x) {
    const int id = ids[j];
    if (id < 0 || id >= vocab) continue;
    float* p = logits + (size_t)r * stride + id;
    const float v = sanitize(*p);                     // same order as the reference: clamp, then penalise
    *p = v > 0.f ? v / pen : v * pen;
  }
}

// logits[r, id] = -inf for the listed ids (no-repeat-n-gram bans computed by the caller).
__global__ void ban_tokens_kernel(float* __restrict__ logits, long stride, int vocab,
                                  const int* __restrict__ ids, const int* __restrict__ id_offsets) {
  const int r = blockIdx.x;
  for (int j = id_offsets[r] + threadIdx.x; j < id_offsets[r + 1]; j += blockDim.x) {
    const int id = ids[j];
    if (id >= 0 && id < vocab) logits[(size_t)r * stride + id] = -INFINITY;
  }
}

}  // namespace cpi

using namespace cpi;

extern "C" int cpi_argmax(const float* logits, long stride, int n_rows, int vocab, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(vocab > 0, "argmax: empty vocabulary");
  count_launch();
  argmax_kernel<<<n_rows, SAMP_NT, 0, stream>>>(logits, stride, vocab, out);
  return check_launch("argmax");
}

extern "C" int cpi_sample(const float* logits, long stride, float* work, int n_rows, int vocab,
                          const float* temperature, const int* top_k, const float* top_p,
                          const float* uniform, int* out, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  CPI_REQUIRE(vocab > 0, "sample: empty vocabulary");
  count_launch();
  sample_kernel<<<n_rows, SAMP_NT, 0, stream>>>(logits, stride, work, vocab, temperature, top_k, top_p, uniform, out);
  return check_launch("sample");
}

extern "C" int cpi_repetition_penalty(float* logits, long stride, int n_rows, int vocab, const int* ids,
                                      const int* id_offsets, const float* penalty, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  count_launch();
  repetition_penalty_kernel<<<n_rows, 256, 0, stream>>>(logits, stride, vocab, ids, id_offsets, penalty);
  return check_launch("repetition_penalty");
}

extern "C" int cpi_ban_tokens(float* logits, long stride, int n_rows, int vocab, const int* ids,
                              const int* id_offsets, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  count_launch();
  ban_tokens_kernel<<<n_rows, 256, 0, stream>>>(logits, stride, vocab, ids, id_offsets);
  return check_launch("ban_tokens");
}
