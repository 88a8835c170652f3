// Attention over the paged key/value cache, general form: any head size that is a multiple of 16 up
// to 256, any number of heads and groups, float32 or bfloat16, prompts and single tokens alike.
//
//   qkv_post   per token and head: optional weightless RMS norm of q and k, rotary position encoding,
//              optional query temperature; writes q to its buffer and k, v into the cache pages.
//   attention  one block per (token, head): scores over the keys the window allows, softmax and the
//              weighted sum of values in float32, keys visited in position order.  A position encoding
//              that acts on the scores hands in a table: score(query at p, key at t) += bias[head][min(p - t,
//              n_dist - 1)].
//
// Formulas (file:line of kurulav1/cpi): per-head norm src/engine/llama4_cpu_engine.cpp:308-317; RoPE pairs
// (d, d + D/2) with angle float(p) * theta_d :167-193, :467; scores, softmax with 1/max(sum, 1e-20) and
// value sum :195-250.  Windows, layers without RoPE, interleaved pairing and the query temperature
// q *= 1 + a * ln(floor((p + 1) / f) + 1) are this library's own.
//
// Cache layout per layer: [page][kv head][slot in page][D]; a sequence's block b (positions
// b*PAGE .. b*PAGE+PAGE-1) lives in page page_table[slot * max_blocks + b].
#include "common.cuh"

namespace cpi {

struct QkvPostParams {
  const void* qkv; long qkv_stride;      // [T, (NH + 2 NKV) D]   (or [T, NH D] when write_kv == 0)
  void* q_out;                           // [T, NH D]
  void* k_cache; void* v_cache;
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  const float* inv_freq;                 // [D/2] or null: no rotation
  int interleaved;
  int qk_norm; int norm_before_rope; float norm_eps;
  int temperature; float floor_scale; float attn_scale;
  int n_heads, n_kv_heads, head_dim, write_kv;
};

template <typename T>
__global__ void qkv_post_kernel(QkvPostParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = p.n_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const int hs = blockIdx.y * (blockDim.x >> 5) + warp;       // head slot
  if (hs >= heads_total) return;
  const int t = blockIdx.x;
  const int D = p.head_dim, half = D >> 1;
  const T* src = reinterpret_cast<const T*>(p.qkv) + (size_t)t * p.qkv_stride + (size_t)hs * D;
  const int pos = p.token_pos[t];
  const bool is_q = hs < p.n_heads;
  const bool is_v = hs >= p.n_heads + p.n_kv_heads;

  T* dst;
  if (is_q) {
    dst = reinterpret_cast<T*>(p.q_out) + ((size_t)t * p.n_heads + hs) * D;
  } else {
    const int kvh = is_v ? hs - p.n_heads - p.n_kv_heads : hs - p.n_heads;
    const int slot = p.seq_slot[p.token_seq[t]];
    const int page = p.page_table[(size_t)slot * p.max_blocks + pos / p.page_size];
    T* base = reinterpret_cast<T*>(is_v ? p.v_cache : p.k_cache);
    dst = base + (((size_t)page * p.n_kv_heads + kvh) * p.page_size + pos % p.page_size) * D;
  }
  if (is_v) {
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
    return;
  }
  float a[4], b[4];                      // pairs lane, lane+32, ... (D <= 256)
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    a[j] = b[j] = 0.f;
    if (i < half) {
      const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
      a[j] = to_f32(src[ia]); b[j] = to_f32(src[ib]);
      ss += a[j] * a[j] + b[j] * b[j];
    }
  }
  if (p.qk_norm && p.norm_before_rope) {
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + p.norm_eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) { a[j] *= inv; b[j] *= inv; }
  }
  if (p.inv_freq) {
    ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j;
      if (i < half) {
        const float ang = (float)pos * p.inv_freq[i];
        float s, c;
        sincosf(ang, &s, &c);
        const float x = a[j], y = b[j];
        a[j] = x * c - y * s;
        b[j] = x * s + y * c;
        ss += a[j] * a[j] + b[j] * b[j];
      }
    }
  }
  if (p.qk_norm && !p.norm_before_rope) {
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + p.norm_eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) { a[j] *= inv; b[j] *= inv; }
  }
  if (is_q && p.temperature) {
    const float sc = 1.0f + p.attn_scale * logf(floorf(((float)pos + 1.0f) / p.floor_scale) + 1.0f);
#pragma unroll
    for (int j = 0; j < 4; ++j) { a[j] *= sc; b[j] *= sc; }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + half;
      dst[ia] = from_f32<T>(a[j]); dst[ib] = from_f32<T>(b[j]);
    }
  }
}

// The same work for bfloat16 heads of 128 with half-split pairs, 16 bytes per lane: a warp takes two heads
// at a time (lanes 0-15 one, 16-31 the other; lane l of a head holds elements 8l .. 8l+7, its rotation
// partner sits 8 lanes away), a block takes a slice of one token's heads and computes the token's 64
// sines and cosines once.  Same formulas as qkv_post_kernel; sums of squares in another order.
__global__ void __launch_bounds__(256) qkv_post_d128_kernel(QkvPostParams p, int heads_per_block) {
  __shared__ float cos_s[64], sin_s[64];
  pdl_launch_dependents();
  // positions and page tables are copied to the device before the step's first kernel and the frequencies
  // are constants: the angles do not wait for the kernel that writes q, k and v
  const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos = p.token_pos[t];
  if (p.inv_freq && tid < 64) {
    float s, c;
    sincosf((float)pos * p.inv_freq[tid], &s, &c);
    cos_s[tid] = c; sin_s[tid] = s;
  }
  pdl_wait();
  __syncthreads();
  const int heads_total = p.n_heads + (p.write_kv ? 2 * p.n_kv_heads : 0);
  const int h_begin = blockIdx.y * heads_per_block, h_end = min(heads_total, h_begin + heads_per_block);
  const int sub = lane >> 4, l = lane & 15;
  const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(p.qkv) + (size_t)t * p.qkv_stride;
  int page = 0;
  if (p.write_kv) {
    const int slot = p.seq_slot[p.token_seq[t]];
    page = p.page_table[(size_t)slot * p.max_blocks + pos / p.page_size];
  }
  const float temp = p.temperature ? 1.0f + p.attn_scale * logf(floorf(((float)pos + 1.0f) / p.floor_scale) + 1.0f) : 1.0f;
  for (int hs = h_begin + 2 * warp + sub; hs < h_end + sub; hs += 2 * (blockDim.x >> 5)) {
    // (all 32 lanes stay in the loop together so that the shuffles below are whole-warp; a lane whose
    // head is past the end computes on zeros and stores nothing)
    const bool live = hs < h_end;
    const bool is_q = hs < p.n_heads, is_v = hs >= p.n_heads + p.n_kv_heads;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (live) raw = *reinterpret_cast<const uint4*>(row + (size_t)hs * 128 + 8 * l);
    __nv_bfloat16* dst = nullptr;
    if (live) {
      if (is_q) {
        dst = reinterpret_cast<__nv_bfloat16*>(p.q_out) + ((size_t)t * p.n_heads + hs) * 128 + 8 * l;
      } else {
        const int kvh = is_v ? hs - p.n_heads - p.n_kv_heads : hs - p.n_heads;
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(is_v ? p.v_cache : p.k_cache);
        dst = base + (((size_t)page * p.n_kv_heads + kvh) * p.page_size + pos % p.page_size) * 128 + 8 * l;
      }
    }
    float x[8];
    {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); x[2 * j] = f.x; x[2 * j + 1] = f.y; }
    }
    const bool rotate = !is_v;                                  // v is copied as it is
    auto group_sum = [&](float v) {
      v += __shfl_xor_sync(0xffffffffu, v, 8); v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 1);
      return v;
    };
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    ss = group_sum(ss);
    if (p.qk_norm && p.norm_before_rope && rotate) {
      const float inv = 1.0f / sqrtf(ss / 128.0f + p.norm_eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= inv;
    }
    if (p.inv_freq) {
      float other[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) other[j] = __shfl_xor_sync(0xffffffffu, x[j], 8);
      if (rotate) {
        const bool first = l < 8;                               // first half: a' = a c - b s; second: b' = a s + b c
        ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = 8 * (l & 7) + j;
          const float c = cos_s[i], sn = sin_s[i];
          x[j] = first ? x[j] * c - other[j] * sn : other[j] * sn + x[j] * c;
          ss += x[j] * x[j];
        }
      }
      ss = group_sum(ss);
    }
    if (p.qk_norm && !p.norm_before_rope && rotate) {
      const float inv = 1.0f / sqrtf(ss / 128.0f + p.norm_eps);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= inv;
    }
    if (is_q && p.temperature) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] *= temp;
    }
    if (live) {
      uint4 o;
      if (is_v) {
        o = raw;
      } else {
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
      }
      *reinterpret_cast<uint4*>(dst) = o;
    }
  }
}

struct AttnParams {
  const void* q; void* out;              // [T, NH D]
  const void* k_cache; const void* v_cache;
  const int* page_table; int max_blocks; int page_size;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  int n_heads, n_kv_heads, head_dim;
  int window_kind, window_size;          // 0 all keys, 1 chunk of window_size, 2 last window_size keys
  float scale;
  const float* score_bias; int n_dist;   // [NH, n_dist] float32 added to the scaled scores by distance, or null
};

__device__ __forceinline__ int window_low(int kind, int size, int pos) {
  if (kind == 1) return (pos / size) * size;
  if (kind == 2) return max(0, pos - size + 1);
  return 0;
}

constexpr int ATT_NT = 128;

template <typename T>
__global__ void __launch_bounds__(ATT_NT) attention_general_kernel(AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float q_s[256];
  __shared__ float p_s[ATT_NT];
  __shared__ size_t off_s[ATT_NT];
  __shared__ float scratch[32];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int D = p.head_dim;
  const int kvh = h / (p.n_heads / p.n_kv_heads);
  const int pos = p.token_pos[t];
  const int slot = p.seq_slot[p.token_seq[t]];
  const int lo = window_low(p.window_kind, p.window_size, pos);
  const T* q = reinterpret_cast<const T*>(p.q) + ((size_t)t * p.n_heads + h) * D;
  for (int i = tid; i < D; i += ATT_NT) q_s[i] = to_f32(q[i]);
  const T* kc = reinterpret_cast<const T*>(p.k_cache);
  const T* vc = reinterpret_cast<const T*>(p.v_cache);
  const int* table = p.page_table + (size_t)slot * p.max_blocks;

  float m_run = -INFINITY, l_run = 0.f, acc0 = 0.f, acc1 = 0.f;
  __syncthreads();
  for (int base = lo; base <= pos; base += ATT_NT) {
    const int kp = base + tid;
    const bool valid = kp <= pos;
    float s = -INFINITY;
    if (valid) {
      const int page = table[kp / p.page_size];
      const size_t off = (((size_t)page * p.n_kv_heads + kvh) * p.page_size + kp % p.page_size) * D;
      off_s[tid] = off;
      const T* kr = kc + off;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(q_s[d], to_f32(kr[d]), dot);
      s = dot * p.scale;
      if (p.score_bias) s += p.score_bias[(size_t)h * p.n_dist + min(pos - kp, p.n_dist - 1)];
    }
    const float m_new = fmaxf(m_run, block_max(s, scratch));
    const float e = valid ? expf(s - m_new) : 0.f;
    p_s[tid] = e;
    const float l_tile = block_sum(e, scratch);       // its barriers also publish p_s and off_s
    const float alpha = expf(m_run - m_new);
    const int nv = min(ATT_NT, pos - base + 1);
    acc0 *= alpha; acc1 *= alpha;
    for (int j = 0; j < nv; ++j) {
      const T* vr = vc + off_s[j];
      const float pj = p_s[j];
      if (tid < D) acc0 = fmaf(pj, to_f32(vr[tid]), acc0);
      if (tid + ATT_NT < D) acc1 = fmaf(pj, to_f32(vr[tid + ATT_NT]), acc1);
    }
    l_run = l_run * alpha + l_tile;
    m_run = m_new;
    __syncthreads();
  }
  const float inv = 1.0f / fmaxf(l_run, 1e-20f);
  T* o = reinterpret_cast<T*>(p.out) + ((size_t)t * p.n_heads + h) * D;
  if (tid < D) o[tid] = from_f32<T>(acc0 * inv);
  if (tid + ATT_NT < D) o[tid + ATT_NT] = from_f32<T>(acc1 * inv);
}

}  // namespace cpi

using namespace cpi;

static int check_head(const char* who, int n_heads, int n_kv_heads, int head_dim) {
  CPI_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
              "%s: %d heads cannot be grouped over %d key/value heads", who, n_heads, n_kv_heads);
  CPI_REQUIRE(head_dim >= 16 && head_dim <= 256 && head_dim % 16 == 0,
              "%s: head size %d is not supported (multiples of 16 from 16 to 256)", who, head_dim);
  return 0;
}

extern "C" int cpi_qkv_post(const void* qkv, long qkv_stride, void* q_out, void* k_cache, void* v_cache,
                            int dtype, const int* page_table, int max_blocks, int page_size,
                            const int* token_seq, const int* token_pos, const int* seq_slot,
                            const float* inv_freq, int interleaved, int qk_norm, int norm_before_rope,
                            float norm_eps, int temperature, float floor_scale, float attn_scale,
                            int n_tokens, int n_heads, int n_kv_heads, int head_dim, int write_kv,
                            cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (check_head("qkv_post", n_heads, n_kv_heads, head_dim)) return 1;
  QkvPostParams p{qkv, qkv_stride, q_out, k_cache, v_cache, page_table, max_blocks, page_size,
                  token_seq, token_pos, seq_slot, inv_freq, interleaved, qk_norm, norm_before_rope,
                  norm_eps, temperature, floor_scale, attn_scale, n_heads, n_kv_heads, head_dim, write_kv};
  const int heads_total = n_heads + (write_kv ? 2 * n_kv_heads : 0);
  auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (dtype == kBF16 && head_dim == 128 && !interleaved && qkv_stride % 8 == 0 && aligned16(qkv) && aligned16(q_out) &&
      (!write_kv || (aligned16(k_cache) && aligned16(v_cache))) && n_tokens <= 65535) {
    // enough blocks for two waves of the GPU, at most one block per 16 heads
    int slices = (2 * sm_count() * 8 + n_tokens - 1) / n_tokens;
    const int max_slices = (heads_total + 15) / 16;
    if (slices > max_slices) slices = max_slices;
    if (slices < 1) slices = 1;
    int per = (heads_total + slices - 1) / slices;
    per = (per + 1) & ~1;                                        // warps take heads two at a time
    dim3 grid_v(n_tokens, (heads_total + per - 1) / per);
    cpi::launch_pdl(qkv_post_d128_kernel, grid_v, 256, 0, stream, p, per);
    return check_launch("qkv_post");
  }
  dim3 grid(n_tokens, (heads_total + 3) / 4);
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(qkv_post_kernel<T>, grid, 128, 0, stream, p));
  return check_launch("qkv_post");
}

extern "C" int cpi_attention_general(const void* q, void* out, const void* k_cache, const void* v_cache,
                                     int dtype, const int* page_table, int max_blocks, int page_size,
                                     const int* token_seq, const int* token_pos, const int* seq_slot,
                                     int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     int window_kind, int window_size, float scale, const float* score_bias,
                                     int n_dist, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (check_head("attention", n_heads, n_kv_heads, head_dim)) return 1;
  CPI_REQUIRE(score_bias == nullptr || n_dist > 0, "attention: a score bias table needs at least one distance");
  CPI_REQUIRE(window_kind == 0 || window_size > 0, "attention: window kind %d needs a size > 0", window_kind);
  CPI_REQUIRE(n_heads <= 65535, "attention: too many heads (%d)", n_heads);
  AttnParams p{q, out, k_cache, v_cache, page_table, max_blocks, page_size, token_seq, token_pos, seq_slot,
               n_heads, n_kv_heads, head_dim, window_kind, window_size, scale, score_bias, n_dist};
  dim3 grid(n_tokens, n_heads);
  CPI_DISPATCH_DTYPE(dtype, T, cpi::launch_pdl(attention_general_kernel<T>, grid, ATT_NT, 0, stream, p));
  return check_launch("attention_general");
}
