// Routing of tokens to experts: router logits and top-k with sigmoid gates, then per-expert row lists.
//
// Reference: router logits = W_r h, the single best expert by a strict '>' scanning upward, so ties go
// to the lowest index, and no gate value (src/engine/llama4_cpu_engine.cpp:256-263; on the host in its
// CUDA engine, src/engine/llama4_cuda_engine_setup.cu:488-519).  Top-k > 1 and the gate
// g = 1 / (1 + exp(-logit)) are this library's own.  Router math is float32 whatever the activation
// dtype, each logit summed in a fixed order so that a token's choice does not depend on its batch.
#include "common.cuh"

namespace cpi {

constexpr int kMaxExperts = 256;

// Router logit = sum over the hidden axis of x * w, float32, in ONE fixed order whichever kernel computes
// it: thread i of 128 adds, element by element, the groups of 8 consecutive elements number i, i + 128,
// i + 256, ...; each thread's sum goes through the warp tree, and the four warp results are added in
// order.  Groups of 8 let every load be 16 bytes (two for float32).
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// the 8 elements of group `g` (zeros beyond `hidden`); `vec`: rows are 16-byte aligned and hidden % 8 == 0
template <typename T> __device__ __forceinline__ void load_group(const T* row, int g, int hidden, bool vec, float (&v)[8]) {
  if (vec) { load8<T>(row + 8 * g, v); return; }
#pragma unroll
  for (int u = 0; u < 8; ++u) v[u] = 8 * g + u < hidden ? to_f32(row[8 * g + u]) : 0.f;
}

// One block per (expert, token) -- for a handful of tokens.
template <typename TH, typename TW>
__global__ void __launch_bounds__(128)
router_logits_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w,
                     float* __restrict__ logits, int hidden, int n_experts, int vec) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  const int e = blockIdx.x, t = blockIdx.y;
  const TH* x = h + (size_t)t * h_stride;
  const TW* wr = w + (size_t)e * hidden;
  const int groups = (hidden + 7) / 8;
  float s = 0.f;
  if (groups <= 8 * 128) {
    // the router's weights are no kernel's output: this thread's (up to eight) groups of them are fetched
    // before the wait on the kernel that writes the activations; same order of additions as below
    float wv[8][8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int g = threadIdx.x + j * 128;
      if (g < groups) load_group<TW>(wr, g, hidden, vec, wv[j]);
    }
    pdl_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int g = threadIdx.x + j * 128;
      if (g < groups) {
        float xv[8];
        load_group<TH>(x, g, hidden, vec, xv);
#pragma unroll
        for (int u = 0; u < 8; ++u) s = fmaf(xv[u], wv[j][u], s);
      }
    }
  } else {
    pdl_wait();
    for (int g = threadIdx.x; g < groups; g += 128) {
      float xv[8], wv[8];
      load_group<TH>(x, g, hidden, vec, xv);
      load_group<TW>(wr, g, hidden, vec, wv);
#pragma unroll
      for (int u = 0; u < 8; ++u) s = fmaf(xv[u], wv[u], s);
    }
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) logits[(size_t)t * n_experts + e] = s;
}

// A block takes TOK tokens and EXP experts at a time -- for many tokens: every loaded activation is used
// EXP times and every loaded weight TOK times.  Same order of additions as above, so the same bits.
template <typename TH, typename TW, int TOK, int EXP>
__global__ void __launch_bounds__(128)
router_logits_tile_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w,
                          float* __restrict__ logits, int n_tokens, int hidden, int n_experts, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float part[4][TOK * EXP];
  const int t0 = blockIdx.x * TOK, e0 = blockIdx.y * EXP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (hidden + 7) / 8;
  float acc[TOK][EXP];
#pragma unroll
  for (int a = 0; a < TOK; ++a)
#pragma unroll
    for (int b = 0; b < EXP; ++b) acc[a][b] = 0.f;
  for (int g = threadIdx.x; g < groups; g += 128) {
    float xv[TOK][8], wv[EXP][8];
#pragma unroll
    for (int a = 0; a < TOK; ++a)            // rows beyond the end repeat the last one; they are not stored
      load_group<TH>(h + (size_t)min(t0 + a, n_tokens - 1) * h_stride, g, hidden, vec, xv[a]);
#pragma unroll
    for (int b = 0; b < EXP; ++b)
      load_group<TW>(w + (size_t)min(e0 + b, n_experts - 1) * hidden, g, hidden, vec, wv[b]);
#pragma unroll
    for (int a = 0; a < TOK; ++a)
#pragma unroll
      for (int b = 0; b < EXP; ++b)
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[a][b] = fmaf(xv[a][u], wv[b][u], acc[a][b]);
  }
#pragma unroll
  for (int a = 0; a < TOK; ++a)
#pragma unroll
    for (int b = 0; b < EXP; ++b) {
      const float v = warp_sum(acc[a][b]);
      if (lane == 0) part[warp][a * EXP + b] = v;
    }
  __syncthreads();
  for (int k = threadIdx.x; k < TOK * EXP; k += 128) {
    const int a = k / EXP, b = k % EXP;
    if (t0 + a < n_tokens && e0 + b < n_experts) {
      float r = 0.f;
      for (int wq = 0; wq < 4; ++wq) r += part[wq][k];
      logits[(size_t)(t0 + a) * n_experts + e0 + b] = r;
    }
  }
}

// The k best logits of one token, ties to the lowest index; gate = sigmoid of the chosen logit.
__device__ __forceinline__ void select_topk(const float* lg, int* idx, float* gate, int n_experts, int top_k, int gate_mode) {
  for (int k = 0; k < top_k; ++k) {
    int best = -1;
    float bv = 0.f;
    for (int e = 0; e < n_experts; ++e) {
      const float v = lg[e];
      if (v != v) continue;                         // NaN never wins
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= (idx[j] == e);
      if (taken) continue;
      if (best < 0 || v > bv) { best = e; bv = v; }
    }
    if (best < 0) {                                 // all NaN: fall back to the lowest free index
      for (int e = 0; e < n_experts && best < 0; ++e) {
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= (idx[j] == e);
        if (!taken) best = e;
      }
      bv = lg[best];
    }
    idx[k] = best;
    gate[k] = gate_mode == 0 ? 1.0f : 1.0f / (1.0f + expf(-bv));
  }
}

// One thread per token.
__global__ void router_select_kernel(const float* __restrict__ logits, int* __restrict__ topk_idx,
                                     float* __restrict__ topk_gate, int n_tokens, int n_experts, int top_k,
                                     int gate_mode) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  select_topk(logits + (size_t)t * n_experts, topk_idx + (size_t)t * top_k, topk_gate + (size_t)t * top_k, n_experts,
              top_k, gate_mode);
}

// A step with few tokens: selection, the per-expert row lists and the gather of the activation rows in
// one launch.  Block r owns sorted row r; every block repeats the (tiny) selection and list building in
// shared memory to learn which token that is, and block 0 also writes the lists out.  Same choices and
// the same stable order as router_select_kernel + moe_lists_kernel.
constexpr int kSmallSlots = 256, kSmallLogits = 4096;
__global__ void __launch_bounds__(128)
moe_route_small_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int top_k, int gate_mode,
                       int* __restrict__ topk_idx, float* __restrict__ topk_gate, int* __restrict__ group_offsets,
                       int* __restrict__ row_token, float* __restrict__ row_scale, int* __restrict__ row_of_slot,
                       const uint4* __restrict__ src, long src_stride16, uint4* __restrict__ dst, int chunks) {
  __shared__ float lg_s[kSmallLogits];
  __shared__ int idx_s[kSmallSlots], rowtok_s[kSmallSlots], offs_s[kMaxExperts + 1];
  __shared__ float gate_s[kSmallSlots];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, M = n_tokens * top_k;
  for (int i = tid; i < n_tokens * n_experts; i += 128) lg_s[i] = logits[i];
  __syncthreads();
  for (int t = tid; t < n_tokens; t += 128)
    select_topk(lg_s + t * n_experts, idx_s + t * top_k, gate_s + t * top_k, n_experts, top_k, gate_mode);
  __syncthreads();
  for (int e = tid; e < n_experts; e += 128) {
    int c = 0;
    for (int q = 0; q < M; ++q) c += idx_s[q] == e;
    offs_s[e + 1] = c;
  }
  __syncthreads();
  if (tid == 0) {
    offs_s[0] = 0;
    for (int e = 0; e < n_experts; ++e) offs_s[e + 1] += offs_s[e];
  }
  __syncthreads();
  const bool writer = blockIdx.x == 0;
  for (int q = tid; q < M; q += 128) {
    const int e = idx_s[q];
    int r = offs_s[e];
    for (int q2 = 0; q2 < q; ++q2) r += idx_s[q2] == e;
    rowtok_s[r] = q / top_k;
    if (writer) {
      row_token[r] = q / top_k;
      row_scale[r] = gate_s[q];
      row_of_slot[q] = r;
      topk_idx[q] = e;
      topk_gate[q] = gate_s[q];
    }
  }
  if (writer)
    for (int e = tid; e <= n_experts; e += 128) group_offsets[e] = offs_s[e];
  __syncthreads();
  const int r = blockIdx.x;
  if (r < M && src) {
    const uint4* from = src + (size_t)rowtok_s[r] * src_stride16;
    uint4* to = dst + (size_t)r * chunks;
    for (int i = tid; i < chunks; i += 128) to[i] = from[i];
  }
}

// Single block of 32 warps: counts, offsets and a stable (token-major) list of rows per expert.
//   group_offsets[e .. e+1]   logical rows of expert e
//   row_token[m]              token whose activation feeds logical row m
//   row_scale[m]              gate of that (token, k)
//   row_of_slot[t*K + k]      logical row that holds (t, k)'s expert output
// A warp owns experts warp, warp + 32, ...; it scans the slots 32 at a time and places the matching
// ones with a ballot, which keeps them in slot order.
constexpr int kListSlotsInSmem = 8192;
__global__ void __launch_bounds__(1024)
moe_lists_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_gate,
                 int* __restrict__ group_offsets, int* __restrict__ row_token,
                 float* __restrict__ row_scale, int* __restrict__ row_of_slot,
                 int n_slots, int top_k, int n_experts) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int counts[kMaxExperts];
  __shared__ int offsets[kMaxExperts + 1];
  __shared__ int idx_s[kListSlotsInSmem];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the choices are scanned twice by every warp: keep them in shared memory when they fit
  const bool staged = n_slots <= kListSlotsInSmem;
  if (staged) {
    for (int s = threadIdx.x; s < n_slots; s += blockDim.x) idx_s[s] = topk_idx[s];
    __syncthreads();
  }
  const int* idx = staged ? idx_s : topk_idx;
  for (int e = warp; e < n_experts; e += 32) {
    int c = 0;
    for (int s0 = 0; s0 < n_slots; s0 += 32) {
      const int s = s0 + lane;
      const bool hit = s < n_slots && idx[s] == e;
      c += __popc(__ballot_sync(0xffffffffu, hit));
    }
    if (lane == 0) counts[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < n_experts; ++i) { offsets[i] = run; run += counts[i]; }
    offsets[n_experts] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) group_offsets[e] = offsets[e];
  for (int e = warp; e < n_experts; e += 32) {
    int m = offsets[e];
    for (int s0 = 0; s0 < n_slots; s0 += 32) {
      const int s = s0 + lane;
      const bool hit = s < n_slots && idx[s] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = m + __popc(mask & ((1u << lane) - 1u));
        row_token[r] = s / top_k;
        row_scale[r] = topk_gate[s];
        row_of_slot[s] = r;
      }
      m += __popc(mask);
    }
  }
}

}  // namespace cpi

using namespace cpi;

// gate_mode: 0 none (gates are 1), 1 sigmoid of the chosen logit
// gate_mode: 0 none (gates are 1), 1 sigmoid of the chosen logit.  `logits` is float32 [n_tokens, n_experts]
// scratch that also serves as the optional output of the router logits.
extern "C" int cpi_router_topk(const void* h, int h_dtype, long h_stride, const void* w, int w_dtype,
                               float* logits, int* topk_idx, float* topk_gate, int n_tokens,
                               int hidden, int n_experts, int top_k, int gate_mode, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_experts >= 1 && n_experts <= kMaxExperts, "router: %d experts (supported: 1..%d)", n_experts, kMaxExperts);
  CPI_REQUIRE(top_k >= 1 && top_k <= n_experts, "router: top-k %d of %d experts", top_k, n_experts);
  CPI_REQUIRE(logits != nullptr, "router: the logits buffer is missing");
  CPI_REQUIRE(n_tokens <= 65535, "router: too many tokens in one launch (%d)", n_tokens);
  const int esz_h = h_dtype == kF32 ? 4 : 2, esz_w = w_dtype == kF32 ? 4 : 2;
  const int vec = hidden % 8 == 0 && (h_stride * esz_h) % 16 == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 &&
                  ((long)hidden * esz_w) % 16 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  if (n_tokens >= 64) {
    constexpr int TOK = 4, EXP = 4;
    dim3 grid((n_tokens + TOK - 1) / TOK, (n_experts + EXP - 1) / EXP);
    CPI_DISPATCH_DTYPE(h_dtype, TH, CPI_DISPATCH_DTYPE(w_dtype, TW,
        (cpi::launch_pdl(router_logits_tile_kernel<TH, TW, TOK, EXP>, grid, 128, 0, stream, (const TH*)h, h_stride, (const TW*)w, logits, n_tokens, hidden, n_experts, vec))));
  } else {
    dim3 grid(n_experts, n_tokens);
    CPI_DISPATCH_DTYPE(h_dtype, TH, CPI_DISPATCH_DTYPE(w_dtype, TW,
        (cpi::launch_pdl(router_logits_kernel<TH, TW>, grid, 128, 0, stream, (const TH*)h, h_stride, (const TW*)w, logits, hidden, n_experts, vec))));
  }
  if (check_launch("router_logits")) return 2;
  if (!topk_idx) return 0;                          // logits only: the caller selects in a later kernel
  cpi::launch_pdl(router_select_kernel, (n_tokens + 127) / 128, 128, 0, stream, logits, topk_idx, topk_gate, n_tokens, n_experts, top_k, gate_mode);
  return check_launch("router_select");
}

// Selection, lists and (when sorted_h is given) the gather for logits already computed: one launch for a
// step with few tokens.  Returns 0 launched, 1 error, -1 when the step is too large for this kernel.
extern "C" int cpi_moe_route_small(const float* logits, int n_tokens, int n_experts, int top_k, int gate_mode,
                                   int* topk_idx, float* topk_gate, int* group_offsets, int* row_token,
                                   float* row_scale, int* row_of_slot, const void* h, long h_stride_bytes,
                                   void* sorted_h, int row_bytes, cudaStream_t stream) {
  if (n_tokens <= 0 || (long)n_tokens * top_k > kSmallSlots || (long)n_tokens * n_experts > kSmallLogits ||
      n_experts > kMaxExperts || top_k < 1 || top_k > n_experts)
    return -1;
  if (sorted_h && (row_bytes % 16 || h_stride_bytes % 16 || (reinterpret_cast<uintptr_t>(h) & 15) ||
                   (reinterpret_cast<uintptr_t>(sorted_h) & 15)))
    return -1;
  cpi::launch_pdl(moe_route_small_kernel, n_tokens * top_k, 128, 0, stream, logits, n_tokens, n_experts, top_k, gate_mode,
                  topk_idx, topk_gate, group_offsets, row_token, row_scale, row_of_slot,
                  sorted_h ? (const uint4*)h : (const uint4*)nullptr, h_stride_bytes / 16, (uint4*)sorted_h, row_bytes / 16);
  return check_launch("moe_route_small") ? 1 : 0;
}

extern "C" int cpi_router_select(const float* logits, int* topk_idx, float* topk_gate, int n_tokens, int n_experts,
                                 int top_k, int gate_mode, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  cpi::launch_pdl(router_select_kernel, (n_tokens + 127) / 128, 128, 0, stream, logits, topk_idx, topk_gate, n_tokens, n_experts, top_k, gate_mode);
  return check_launch("router_select");
}

extern "C" int cpi_moe_lists(const int* topk_idx, const float* topk_gate, int* group_offsets, int* row_token,
                             float* row_scale, int* row_of_slot, int n_tokens, int top_k, int n_experts,
                             cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_experts >= 1 && n_experts <= kMaxExperts, "moe_lists: %d experts (supported: 1..%d)", n_experts, kMaxExperts);
  cpi::launch_pdl(moe_lists_kernel, 1, 1024, 0, stream, topk_idx, topk_gate, group_offsets, row_token, row_scale,
                                              row_of_slot, n_tokens * top_k, top_k, n_experts);
  return check_launch("moe_lists");
}
