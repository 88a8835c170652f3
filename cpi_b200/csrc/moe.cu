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

// One block per (expert, token): its threads stride over the hidden axis, then a fixed-order block sum.
template <typename TH, typename TW>
__global__ void __launch_bounds__(128)
router_logits_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w,
                     float* __restrict__ logits, int hidden, int n_experts) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int e = blockIdx.x, t = blockIdx.y;
  const TH* x = h + (size_t)t * h_stride;
  const TW* wr = w + (size_t)e * hidden;
  float s = 0.f;
#pragma unroll 8
  for (int i = threadIdx.x; i < hidden; i += 128) s = fmaf(to_f32(x[i]), to_f32(wr[i]), s);
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) logits[(size_t)t * n_experts + e] = s;
}

// The same sums for many tokens: one block per token keeps the token's row in registers and visits the
// experts one after the other.  Thread i again sums elements i, i + 128, ... and the block sum is the
// same, so a logit has the same bits whichever of the two kernels computed it.
template <typename TH, typename TW>
__global__ void __launch_bounds__(128)
router_logits_rows_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w,
                          float* __restrict__ logits, int hidden, int n_experts) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  constexpr int PER = 64;                             // up to 8192 hidden elements in registers
  const int t = blockIdx.x;
  const TH* x = h + (size_t)t * h_stride;
  float xv[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int i = threadIdx.x + j * 128;
    xv[j] = i < hidden ? to_f32(x[i]) : 0.f;
  }
  for (int e = 0; e < n_experts; ++e) {
    const TW* wr = w + (size_t)e * hidden;
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * 128;
      if (i < hidden) s = fmaf(xv[j], to_f32(wr[i]), s);
    }
    s = block_sum(s, scratch);
    if (threadIdx.x == 0) logits[(size_t)t * n_experts + e] = s;
  }
}

// One thread per token: the k best logits, ties to the lowest index; gate = sigmoid of the chosen logit.
__global__ void router_select_kernel(const float* __restrict__ logits, int* __restrict__ topk_idx,
                                     float* __restrict__ topk_gate, int n_tokens, int n_experts, int top_k,
                                     int gate_mode) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const float* lg = logits + (size_t)t * n_experts;
  int* idx = topk_idx + (size_t)t * top_k;
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
    topk_gate[(size_t)t * top_k + k] = gate_mode == 0 ? 1.0f : 1.0f / (1.0f + expf(-bv));
  }
}

// Single block of 32 warps: counts, offsets and a stable (token-major) list of rows per expert.
//   group_offsets[e .. e+1]   logical rows of expert e
//   row_token[m]              token whose activation feeds logical row m
//   row_scale[m]              gate of that (token, k)
//   row_of_slot[t*K + k]      logical row that holds (t, k)'s expert output
// A warp owns experts warp, warp + 32, ...; it scans the slots 32 at a time and places the matching
// ones with a ballot, which keeps them in slot order.
__global__ void __launch_bounds__(1024)
moe_lists_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_gate,
                 int* __restrict__ group_offsets, int* __restrict__ row_token,
                 float* __restrict__ row_scale, int* __restrict__ row_of_slot,
                 int n_slots, int top_k, int n_experts) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int counts[kMaxExperts];
  __shared__ int offsets[kMaxExperts + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < n_experts; e += 32) {
    int c = 0;
    for (int s0 = 0; s0 < n_slots; s0 += 32) {
      const int s = s0 + lane;
      const bool hit = s < n_slots && topk_idx[s] == e;
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
      const bool hit = s < n_slots && topk_idx[s] == e;
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
  if (n_tokens >= 128 && hidden <= 64 * 128) {
    CPI_DISPATCH_DTYPE(h_dtype, TH, CPI_DISPATCH_DTYPE(w_dtype, TW,
        (cpi::launch_pdl(router_logits_rows_kernel<TH, TW>, n_tokens, 128, 0, stream, (const TH*)h, h_stride, (const TW*)w, logits, hidden, n_experts))));
  } else {
    dim3 grid(n_experts, n_tokens);
    CPI_DISPATCH_DTYPE(h_dtype, TH, CPI_DISPATCH_DTYPE(w_dtype, TW,
        (cpi::launch_pdl(router_logits_kernel<TH, TW>, grid, 128, 0, stream, (const TH*)h, h_stride, (const TW*)w, logits, hidden, n_experts))));
  }
  if (check_launch("router_logits")) return 2;
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
