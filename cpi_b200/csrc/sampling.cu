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
  if (vocab % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // 16-byte loads, several in flight: one block reads the whole row.  A thread meets its elements in
    // increasing index order, so `>` keeps its smallest index; the block then prefers the smallest index.
    const float4* r4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
    for (int i = threadIdx.x; i < vocab / 4; i += SAMP_NT) {
      const float4 v = r4[i];
      if (v.x > best) { best = v.x; bi = 4 * i; }
      if (v.y > best) { best = v.y; bi = 4 * i + 1; }
      if (v.z > best) { best = v.z; bi = 4 * i + 2; }
      if (v.w > best) { best = v.w; bi = 4 * i + 3; }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += SAMP_NT) {
      const float v = row[i];
      if (v > best) { best = v; bi = i; }             // strided scan keeps the smallest index per thread
    }
  }
  block_argmax(best, bi, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// Visits every element of a row: four neighbouring elements per thread and iteration through 16-byte loads
// when the row allows it (a single block reads a whole vocabulary: what counts is how many loads it has in
// flight), else one by one.  body(index, value).
template <typename F>
__device__ __forceinline__ void for_row(const float* __restrict__ src, int n, bool vec, F body) {
  if (vec) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
#pragma unroll 4
    for (int i = threadIdx.x; i < n / 4; i += SAMP_NT) {
      const float4 v = s4[i];
      body(4 * i, v.x); body(4 * i + 1, v.y); body(4 * i + 2, v.z); body(4 * i + 3, v.w);
    }
  } else {
    for (int i = threadIdx.x; i < n; i += SAMP_NT) body(i, src[i]);
  }
}

constexpr int SAMP_CAND = 2048;                       // candidates the block sorts in shared memory

// One block per row.  `work` is a float32 [rows, vocab] scratch; afterwards it holds the row's weights
// e = exp(logit / T - max).
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
  __shared__ unsigned cand_u[SAMP_CAND], sel[3];      // cand_u doubles as the histogram of the fallback
  __shared__ int cand_i[SAMP_CAND], n_cand;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * stride;
  float* w = work + (size_t)r * vocab;
  const bool vec = vocab % 4 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
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
  for_row(row, vocab, vec, [&](int, float x) { mx = fmaxf(mx, sanitize(x) * inv_t); });
  mx = block_max(mx, scratch);
  if (mx == -INFINITY) { if (tid == 0) out[r] = 0; return; }
  float sum = 0.f, tmax = 0.f;
  for_row(row, vocab, vec, [&](int i, float x) {
    const float v = sanitize(x) * inv_t;
    const float e = v == -INFINITY ? 0.f : expf(v - mx);
    w[i] = e;
    sum += e;
    tmax = fmaxf(tmax, e);
  });
  sum = block_sum(sum, scratch);
  const float inv_sum = 1.0f / sum;
  const int k = max(1, min(min(top_k[r], vocab), 256));
  const float tp = top_p[r];
  const bool use_p = tp > 0.f && tp < 1.f;
  // ---- the k largest weights, largest first, equal ones by index.  The weights are non-negative floats,
  // so their bit patterns order like the values.
  // A floor first: the k-th largest of the 1024 per-thread maxima is the weight of some entry with at least
  // k entries at or above it, so the k-th largest overall is no smaller.  The entries at or above the floor
  // (usually a few hundred) are gathered in one pass and sorted in shared memory.  Only if there are more
  // of them than fit (thousands of equal logits) does a radix select over the row find the k-th largest
  // pattern t (11 + 11 + 10 bits, a histogram pass each), after which everything above t is kept and of
  // the entries equal to t the ones with the lowest indices. ----
  cand_u[tid] = __float_as_uint(tmax);
  __syncthreads();
  for (int size = 2; size <= SAMP_NT; size <<= 1)
    for (int st = size >> 1; st > 0; st >>= 1) {
      const int partner = tid ^ st;
      if (partner > tid) {
        const bool down = (tid & size) == 0;          // largest first
        const unsigned a = cand_u[tid], b = cand_u[partner];
        if ((a < b) == down) { cand_u[tid] = b; cand_u[partner] = a; }
      }
      __syncthreads();
    }
  const unsigned floor_bits = max(cand_u[min(k, SAMP_NT) - 1], 1u);     // (weights of zero are never kept)
  __syncthreads();
  if (tid == 0) n_cand = 0;
  for (int i = tid; i < SAMP_CAND; i += SAMP_NT) { cand_u[i] = 0; cand_i[i] = 0x7fffffff; }
  __syncthreads();
  for_row(w, vocab, vec, [&](int i, float e) {
    const unsigned u = __float_as_uint(e);
    if (u >= floor_bits) {
      const int slot = atomicAdd(&n_cand, 1);
      if (slot < SAMP_CAND) { cand_u[slot] = u; cand_i[slot] = i; }
    }
  });
  __syncthreads();
  const int n_above = n_cand;
  __syncthreads();
  if (n_above > SAMP_CAND) {
    unsigned* hist = cand_u;
    unsigned prefix = 0, mask = 0;
    int need = k;                                     // entries still to be found among those matching the prefix
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
      const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
      const unsigned bins = pass == 2 ? 1024u : 2048u;
      for (int i = tid; i < 2048; i += SAMP_NT) hist[i] = 0;
      __syncthreads();
      for_row(w, vocab, vec, [&](int, float e) {
        const unsigned u = __float_as_uint(e);
        if (u >= floor_bits && (u & mask) == prefix) atomicAdd(&hist[(u >> shift) & (bins - 1)], 1u);
      });
      __syncthreads();
      if (tid == 0) {
        int acc = 0, b = (int)bins - 1;
        for (; b > 0; --b) {
          if (acc + (int)hist[b] >= need) break;
          acc += (int)hist[b];
        }
        sel[0] = (unsigned)b;
        sel[1] = (unsigned)(need - acc);
        sel[2] = hist[b];
      }
      __syncthreads();
      prefix |= sel[0] << shift;
      mask |= (bins - 1) << shift;
      need = (int)sel[1];
      __syncthreads();
    }
    const unsigned t = prefix;                        // the k-th largest pattern
    const int n_equal = (int)sel[2];                  // entries equal to t
    if (tid == 0) n_cand = 0;
    for (int i = tid; i < SAMP_CAND; i += SAMP_NT) { cand_u[i] = 0; cand_i[i] = 0x7fffffff; }
    __syncthreads();
    for_row(w, vocab, vec, [&](int i, float e) {
      const unsigned u = __float_as_uint(e);
      if (u >= floor_bits && (u > t || (u == t && n_equal <= need))) {     // all of the equals are wanted: any order
        const int slot = atomicAdd(&n_cand, 1);
        if (slot < SAMP_CAND) { cand_u[slot] = u; cand_i[slot] = i; }
      }
    });
    __syncthreads();
    if (n_equal > need && t >= floor_bits) {
      // more equals than places: the lowest indices, found by an ordered scan over consecutive indices
      int taken = 0;
      for (int base = 0; base < vocab && taken < need; base += SAMP_NT) {
        const int i = base + tid;
        const bool hit = i < vocab && __float_as_uint(w[i]) == t;
        const unsigned bal = __ballot_sync(0xffffffffu, hit);
        const int lane = tid & 31, warp = tid >> 5;
        if (lane == 0) si[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int q = 0; q < SAMP_NT / 32; ++q) { if (q < warp) before += si[q]; total += si[q]; }
        const int rank = taken + before + __popc(bal & ((1u << lane) - 1u));
        if (hit && rank < need) {
          const int slot = atomicAdd(&n_cand, 1);
          if (slot < SAMP_CAND) { cand_u[slot] = t; cand_i[slot] = i; }
        }
        taken += total;
        __syncthreads();
      }
    }
    __syncthreads();
  }
  // bitonic sort of the candidate array (pattern descending, index ascending); empty places sink to the end
  for (int size = 2; size <= SAMP_CAND; size <<= 1) {
    for (int st = size >> 1; st > 0; st >>= 1) {
#pragma unroll
      for (int rep = 0; rep < SAMP_CAND / (2 * SAMP_NT); ++rep) {
        const int q = tid + rep * SAMP_NT;                       // which compare-exchange
        const int lo = ((q & ~(st - 1)) << 1) | (q & (st - 1));  // its lower element
        const int hi = lo | st;
        const bool up = (lo & size) == 0;                        // this pair sorts towards "best first"
        const unsigned ua = cand_u[lo], ub = cand_u[hi];
        const int ia = cand_i[lo], ib = cand_i[hi];
        const bool a_first = ua > ub || (ua == ub && ia < ib);
        if (a_first != up) { cand_u[lo] = ub; cand_u[hi] = ua; cand_i[lo] = ib; cand_i[hi] = ia; }
      }
      __syncthreads();
    }
  }
  if (tid == 0) {
    // walk them in descending order; stop once the kept mass reaches top_p (the crossing token is kept)
    int n_kept = 0;
    float kept_sum = 0.f;
    for (int j = 0; j < k; ++j) {
      const float e = __uint_as_float(cand_u[j]);
      if (!(e > 0.f)) break;
      kept_p[n_kept] = e * inv_sum;
      kept_sum += e * inv_sum;
      ++n_kept;
      if (use_p && kept_sum >= tp) break;
    }
    if (n_kept == 0) { out[r] = 0; return; }
    float renorm = 0.f;
    for (int j = 0; j < n_kept; ++j) renorm += kept_p[j];
    const float u = uniform[r];
    float run = 0.f;
    int pick = cand_i[n_kept - 1];
    for (int j = 0; j < n_kept; ++j) {
      run += kept_p[j] / renorm;
      if (u <= run) { pick = cand_i[j]; break; }
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
