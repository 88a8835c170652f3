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

// one block per token: the warps share the experts, thread 0 picks the top k
constexpr int ROUTER_WARPS = 8;

template <typename TH, typename TW>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_topk_kernel(const TH* __restrict__ h, long h_stride, const TW* __restrict__ w,
                   float* __restrict__ logits_out, int* __restrict__ topk_idx,
                   float* __restrict__ topk_gate, int n_tokens, int hidden, int n_experts,
                   int top_k, int gate_mode) {
  __shared__ float lg[kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const TH* x = h + (size_t)t * h_stride;
  for (int e = warp; e < n_experts; e += ROUTER_WARPS) {
    const TW* wr = w + (size_t)e * hidden;
    float s = 0.f;                                  // lane-strided partial sums, then a fixed warp tree
#pragma unroll 4
    for (int i = lane; i < hidden; i += 32) s = fmaf(to_f32(x[i]), to_f32(wr[i]), s);
    s = warp_sum(s);
    if (lane == 0) {
      lg[e] = s;
      if (logits_out) logits_out[(size_t)t * n_experts + e] = s;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 0; k < top_k; ++k) {
      int best = -1;
      for (int e = 0; e < n_experts; ++e) {
        const float v = lg[e];
        if (v != v) continue;                       // NaN never wins
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= (topk_idx[(size_t)t * top_k + j] == e);
        if (taken) continue;
        if (best < 0 || v > lg[best]) best = e;
      }
      if (best < 0) {                               // all NaN: fall back to the lowest free index
        for (int e = 0; e < n_experts && best < 0; ++e) {
          bool taken = false;
          for (int j = 0; j < k; ++j) taken |= (topk_idx[(size_t)t * top_k + j] == e);
          if (!taken) best = e;
        }
      }
      topk_idx[(size_t)t * top_k + k] = best;
      const float r = lg[best];
      topk_gate[(size_t)t * top_k + k] = gate_mode == 0 ? 1.0f : 1.0f / (1.0f + expf(-r));
    }
  }
}

// Single block: counts, offsets and a stable (token-major) list of rows per expert.
//   group_offsets[e .. e+1]   logical rows of expert e
//   row_token[m]              token whose activation feeds logical row m
//   row_scale[m]              gate of that (token, k)
//   row_of_slot[t*K + k]      logical row that holds (t, k)'s expert output
__global__ void moe_lists_kernel(const int* __restrict__ topk_idx, const float* __restrict__ topk_gate,
                                 int* __restrict__ group_offsets, int* __restrict__ row_token,
                                 float* __restrict__ row_scale, int* __restrict__ row_of_slot,
                                 int n_slots, int top_k, int n_experts) {
  __shared__ int counts[kMaxExperts];
  __shared__ int offsets[kMaxExperts + 1];
  const int e = threadIdx.x;
  if (e < n_experts) {
    int c = 0;
    for (int s = 0; s < n_slots; ++s) c += (topk_idx[s] == e);
    counts[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < n_experts; ++i) { offsets[i] = run; run += counts[i]; }
    offsets[n_experts] = run;
  }
  __syncthreads();
  if (e <= n_experts) group_offsets[e] = offsets[e];
  if (e < n_experts) {
    int m = offsets[e];
    for (int s = 0; s < n_slots; ++s) {
      if (topk_idx[s] == e) {
        row_token[m] = s / top_k;
        row_scale[m] = topk_gate[s];
        row_of_slot[s] = m;
        ++m;
      }
    }
  }
}

}  // namespace cpi

using namespace cpi;

// gate_mode: 0 none (gates are 1), 1 sigmoid of the chosen logit
extern "C" int cpi_router_topk(const void* h, int h_dtype, long h_stride, const void* w, int w_dtype,
                               float* logits_out, int* topk_idx, float* topk_gate, int n_tokens,
                               int hidden, int n_experts, int top_k, int gate_mode, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_experts >= 1 && n_experts <= kMaxExperts, "router: %d experts (supported: 1..%d)", n_experts, kMaxExperts);
  CPI_REQUIRE(top_k >= 1 && top_k <= n_experts, "router: top-k %d of %d experts", top_k, n_experts);
  CPI_DISPATCH_DTYPE(h_dtype, TH, CPI_DISPATCH_DTYPE(w_dtype, TW,
      (router_topk_kernel<TH, TW><<<n_tokens, ROUTER_WARPS * 32, 0, stream>>>(
          (const TH*)h, h_stride, (const TW*)w, logits_out, topk_idx, topk_gate, n_tokens, hidden,
          n_experts, top_k, gate_mode))));
  return check_launch("router_topk");
}

extern "C" int cpi_moe_lists(const int* topk_idx, const float* topk_gate, int* group_offsets, int* row_token,
                             float* row_scale, int* row_of_slot, int n_tokens, int top_k, int n_experts,
                             cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_experts >= 1 && n_experts <= kMaxExperts, "moe_lists: %d experts (supported: 1..%d)", n_experts, kMaxExperts);
  int threads = ((n_experts + 1 + 31) / 32) * 32;
  moe_lists_kernel<<<1, threads, 0, stream>>>(topk_idx, topk_gate, group_offsets, row_token, row_scale,
                                              row_of_slot, n_tokens * top_k, top_k, n_experts);
  return check_launch("moe_lists");
}
