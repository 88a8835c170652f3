// Decode attention in bfloat16: one new token per sequence against its paged cache, split over the keys.
//
// A block serves one (split, key/value head, sequence): the G query heads that share the key/value head
// form the rows of a 16-row MMA tile, so every key and value byte is read once per group and not once
// per head.  Keys and values arrive page by page (64 positions x D) through cp.async into a
// double-buffered, XOR-swizzled shared-memory tile; each of the four warps owns 16 keys of the page
// and runs its own online softmax (scores S = Q K^T and the product P V on mma.sync m16n8k16 with
// float32 accumulators; a 5..16-row problem is below the 64-row minimum of tcgen05, and the kernel is
// bound by the cache bytes, not by the tensor pipe).  Warps, then splits, are merged with the usual
// (max, sum) rescaling; with one split the block writes the output itself, otherwise it writes
// float32 partials that a small second kernel combines.
//
// Reference: gqa_decode_kernel (src/kernels/kernels_attention_decode.cu:868-951) visits one key per
// iteration with three block barriers each; formulas as in src/engine/llama4_cpu_engine.cpp:195-250.
// Positions outside [window low, pos] are masked, and their tile rows are zero-filled so that stale
// page contents can never reach the result.
#include "common.cuh"

namespace cpi {
namespace dec {

constexpr int PAGE = 64;
constexpr int NT = 128;

struct Params {
  const __nv_bfloat16* q; __nv_bfloat16* out;      // [B, NH, D]  (token t = sequence t of the step)
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* page_table; int max_blocks;
  const int* token_seq; const int* token_pos; const int* seq_slot;
  int n_heads, n_kv_heads;
  int window_kind, window_size;
  float scale_log2;                                 // softmax scale * log2(e)
  int n_splits;
  float* part_o; float* part_ml;                    // [T, NH, splits, D], [T, NH, splits, 2]
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int n = valid ? 16 : 0;                     // 0 source bytes: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ int window_low(int kind, int size, int pos) {
  if (kind == 1) return (pos / size) * size;
  if (kind == 2) return max(0, pos - size + 1);
  return 0;
}

// shared tile: PAGE rows of D bf16; 16-byte chunk c of row r is stored at chunk c ^ (r & 7)
template <int D> __device__ __forceinline__ int tile_off(int row, int chunk) {
  return row * D + ((chunk ^ (row & 7)) << 3);
}

// out[th, :] = sum_s w_s O_s / sum_s w_s l_s,  w_s = 2^(m_s - max m), for one (token, head); at most
// kMaxSplits splits.  All threads of the block call it (it has barriers); the weights are computed once,
// in parallel, and the sum over splits keeps eight loads in flight.  (Merging inside the attention kernel, by
// the block that takes a group's last ticket, was measured slower at every batch size: one block then
// merges all the heads of its group one after the other.)
constexpr int kMaxSplits = 256;
struct CombineSmem { float w[kMaxSplits], wl[kMaxSplits], red[4]; };
__device__ __forceinline__ void combine_head(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                             __nv_bfloat16* __restrict__ out, size_t th, int n_splits, int D,
                                             CombineSmem& sm) {
  const int tid = threadIdx.x, n_warps = blockDim.x >> 5;
  const float2* ml = reinterpret_cast<const float2*>(part_ml) + th * n_splits;
  const float* po = part_o + th * n_splits * D;
  if (n_splits <= 32 && D <= (int)blockDim.x) {
    // Few splits: every thread fetches all (m, l) pairs and its own feature of every part at once (one
    // round trip to the L2 instead of two or more), then does the arithmetic alone; no barrier.
    float2 mlv[32];
    float v[32];
    const bool mine = tid < D;
#pragma unroll
    for (int s = 0; s < 32; ++s) {
      mlv[s] = s < n_splits ? __ldcg(ml + s) : make_float2(-1e30f, 0.f);
      v[s] = (s < n_splits && mine) ? __ldcg(po + (size_t)s * D + tid) : 0.f;
    }
    float M = -1e30f;
#pragma unroll
    for (int s = 0; s < 32; ++s) M = fmaxf(M, mlv[s].x);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int s = 0; s < 32; ++s) {
      if (s < n_splits) {
        const float f = exp2f(mlv[s].x - M);
        L += f * mlv[s].y;
        acc += f * v[s];
      }
    }
    if (mine) out[th * D + tid] = __float2bfloat16_rn(acc / fmaxf(L, 1e-20f));
    return;
  }
  float2 part[kMaxSplits / 64];                       // blockDim.x >= 64
  float m = -1e30f;
#pragma unroll
  for (int j = 0; j < kMaxSplits / 64; ++j) {
    const int s = tid + j * blockDim.x;
    part[j] = s < n_splits ? __ldcg(ml + s) : make_float2(-1e30f, 0.f);
    m = fmaxf(m, part[j].x);
  }
  m = warp_max(m);
  __syncthreads();                                    // the previous head's readers are done with sm
  if ((tid & 31) == 0) sm.red[tid >> 5] = m;
  __syncthreads();
  float M = sm.red[0];
  for (int w = 1; w < n_warps; ++w) M = fmaxf(M, sm.red[w]);
#pragma unroll
  for (int j = 0; j < kMaxSplits / 64; ++j) {
    const int s = tid + j * blockDim.x;
    if (s < n_splits) {
      const float f = exp2f(part[j].x - M);
      sm.w[s] = f;
      sm.wl[s] = f * part[j].y;
    }
  }
  __syncthreads();
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) L += sm.wl[s];
  for (int d = tid; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s0 = 0; s0 < n_splits; s0 += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = s0 + j < n_splits ? __ldcg(po + (size_t)(s0 + j) * D + d) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) if (s0 + j < n_splits) acc += sm.w[s0 + j] * v[j];
    }
    out[th * D + d] = __float2bfloat16_rn(acc / fmaxf(L, 1e-20f));
  }
}

template <int D>
__global__ void __launch_bounds__(NT) attention_decode_kernel(Params p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CH = D / 8;                 // 16-byte chunks per row
  constexpr int KS = D / 16;                // k-steps of Q K^T
  constexpr int NO = D / 8;                 // n-tiles of the output
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [2][PAGE][D]
  __nv_bfloat16* v_s = k_s + 2 * PAGE * D;                                     // [2][PAGE][D]

  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.n_heads / p.n_kv_heads;
  const int pos = p.token_pos[t];
  const int slot = p.seq_slot[p.token_seq[t]];
  const int lo = window_low(p.window_kind, p.window_size, pos);
  const int* table = p.page_table + (size_t)slot * p.max_blocks;
  const int b_lo = lo / PAGE, b_hi = pos / PAGE;
  const int n_blocks = b_hi - b_lo + 1;
  const int per = (n_blocks + p.n_splits - 1) / p.n_splits;
  const int b_begin = b_lo + split * per;
  const int b_end = min(b_hi + 1, b_begin + per);

  // ---- Q fragments: rows = the group's heads (rows >= G are zero) ----
  const int r0 = lane >> 2, j = lane & 3;
  uint32_t qa[KS][4];
  {
    const __nv_bfloat16* qb = p.q + ((size_t)t * p.n_heads + (size_t)kvh * G) * D;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + 2 * j;
      qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)r0 * D + d) : 0u;
      qa[ks][1] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)(r0 + 8) * D + d) : 0u;
      qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)r0 * D + d + 8) : 0u;
      qa[ks][3] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + (size_t)(r0 + 8) * D + d + 8) : 0u;
    }
  }

  auto load_tile = [&](int blk, int buf) {
    const int page = table[blk];
    const size_t base = ((size_t)page * p.n_kv_heads + kvh) * (size_t)(PAGE * D);
    const int first = blk * PAGE;
#pragma unroll
    for (int i = 0; i < PAGE * CH / NT; ++i) {
      const int c = tid + i * NT;
      const int row = c / CH, ch = c % CH;
      const int kp = first + row;
      const bool valid = kp >= lo && kp <= pos;
      const size_t g = base + (size_t)row * D + ch * 8;
      cp_async16(k_s + buf * PAGE * D + tile_off<D>(row, ch), p.k_cache + g, valid);
      cp_async16(v_s + buf * PAGE * D + tile_off<D>(row, ch), p.v_cache + g, valid);
    }
    cp_async_commit();
  };

  float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};
  float o[NO][4];
#pragma unroll
  for (int i = 0; i < NO; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  if (b_begin < b_end) load_tile(b_begin, 0);
  for (int blk = b_begin; blk < b_end; ++blk) {
    const int buf = (blk - b_begin) & 1;
    if (blk + 1 < b_end) { load_tile(blk + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const __nv_bfloat16* kt = k_s + buf * PAGE * D;
    const __nv_bfloat16* vt = v_s + buf * PAGE * D;
    const int key0 = warp * 16;                       // this warp's 16 keys of the page

    // ---- S = Q K^T for 16 keys: two n-tiles of 8 ----
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      // matrices: (keys 0-7, dims 16ks..+7), (keys 0-7, dims +8..15), (keys 8-15, dims ..+7), (keys 8-15, +8..15)
      const int row = key0 + (lane & 7) + ((lane >> 4) << 3);
      const int ch = ks * 2 + ((lane >> 3) & 1);
      uint32_t b[4];
      ldmatrix_x4(b, kt + tile_off<D>(row, ch));
      mma_bf16(s[0], qa[ks], b[0], b[1]);
      mma_bf16(s[1], qa[ks], b[2], b[3]);
    }
    // ---- mask, online softmax (rows r0 and r0 + 8; this thread holds keys 2j, 2j+1 of each n-tile) ----
    const int kbase = blk * PAGE + key0 + 2 * j;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kp = kbase + nt * 8 + (e & 1);
        const bool valid = kp >= lo && kp <= pos;
        s[nt][e] = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      alpha[h] = exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
    }
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[nt][e] = exp2f(s[nt][e] - m_run[e >> 1]);
        ls[e >> 1] += s[nt][e];
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + ls[h];
#pragma unroll
    for (int i = 0; i < NO; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
    // ---- O += P V: P (16 rows x 16 keys) from the score registers ----
    uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                      pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
    for (int nt2 = 0; nt2 < NO / 2; ++nt2) {
      // transposed matrices: (keys 0-7, dims 16nt2..+7), (keys 8-15, same dims), (keys 0-7, dims +8..15), (keys 8-15, ...)
      const int row = key0 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int ch = nt2 * 2 + (lane >> 4);
      uint32_t b[4];
      ldmatrix_x4_trans(b, vt + tile_off<D>(row, ch));
      mma_bf16(o[2 * nt2], pa, b[0], b[1]);
      mma_bf16(o[2 * nt2 + 1], pa, b[2], b[3]);
    }
    __syncthreads();                                  // the buffer is loaded again two pages later
  }
  // l is a sum over this thread's columns only: complete it over the quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  // ---- merge the four warps through shared memory (reusing the tiles) ----
  float* mo = reinterpret_cast<float*>(smem_raw);              // [4 warps][16 rows][D]
  float* mm = mo + 4 * 16 * D;                                 // [4][16]
  float* ml = mm + 64;                                         // [4][16]
#pragma unroll
  for (int i = 0; i < NO; ++i) {
    const int d = i * 8 + 2 * j;
    float* a = mo + ((size_t)warp * 16 + r0) * D + d;
    a[0] = o[i][0]; a[1] = o[i][1];
    a[8 * D] = o[i][2]; a[8 * D + 1] = o[i][3];
  }
  if (j == 0) {
    mm[warp * 16 + r0] = m_run[0]; mm[warp * 16 + r0 + 8] = m_run[1];
    ml[warp * 16 + r0] = l_run[0]; ml[warp * 16 + r0 + 8] = l_run[1];
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += NT) {
    const int g = idx / D, d = idx % D;
    float M = -1e30f;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 16 + g]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(mm[w * 16 + g] - M);
      acc += f * mo[((size_t)w * 16 + g) * D + d];
      L += f * ml[w * 16 + g];
    }
    const int head = kvh * G + g;
    if (p.n_splits == 1) {
      p.out[((size_t)t * p.n_heads + head) * D + d] = __float2bfloat16_rn(acc / fmaxf(L, 1e-20f));
    } else {
      const size_t pi = ((size_t)t * p.n_heads + head) * p.n_splits + split;
      p.part_o[pi * D + d] = acc;
      if (d == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = L; }
    }
  }
}

__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         __nv_bfloat16* __restrict__ out, int n_splits, int D) {
  __shared__ CombineSmem sm;
  pdl_launch_dependents();
  pdl_wait();
  combine_head(part_o, part_ml, out, blockIdx.x, n_splits, D, sm);
}

}  // namespace dec
}  // namespace cpi

using namespace cpi;

// Returns 0 and launches, or 1 with a message.  The caller checks `cpi_attention_decode_supported` first.
extern "C" int cpi_attention_decode_supported(int n_heads, int n_kv_heads, int head_dim, int page_size) {
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
  return (head_dim == 64 || head_dim == 128) && page_size == dec::PAGE && n_heads / n_kv_heads <= 16;
}

// q, out [T, NH, D] bfloat16, one token per sequence.  part_o needs T*NH*splits*D floats, part_ml
// T*NH*splits*2 floats (both unused when n_splits == 1).
extern "C" int cpi_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                    const int* page_table, int max_blocks, int page_size, const int* token_seq,
                                    const int* token_pos, const int* seq_slot, int n_tokens, int n_heads,
                                    int n_kv_heads, int head_dim, int window_kind, int window_size, float scale,
                                    int n_splits, float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(cpi_attention_decode_supported(n_heads, n_kv_heads, head_dim, page_size),
              "attention_decode: unsupported shape (heads %d/%d, head size %d, page %d)", n_heads, n_kv_heads, head_dim, page_size);
  CPI_REQUIRE(window_kind == 0 || window_size > 0, "attention_decode: window kind %d needs a size > 0", window_kind);
  CPI_REQUIRE(n_splits >= 1 && n_splits <= dec::kMaxSplits && n_tokens <= 65535, "attention_decode: bad grid (%d splits of at most %d, %d tokens)", n_splits, dec::kMaxSplits, n_tokens);
  CPI_REQUIRE(n_splits == 1 || (part_o && part_ml), "attention_decode: split scratch is missing");
  dec::Params p{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                page_table, max_blocks, token_seq, token_pos, seq_slot, n_heads, n_kv_heads, window_kind, window_size,
                scale * 1.4426950408889634f, n_splits, part_o, part_ml};
  dim3 grid(n_splits, n_kv_heads, n_tokens);
  const int smem_tiles = 4 * dec::PAGE * head_dim * 2;
  const int smem_merge = (4 * 16 * head_dim + 128) * 4;
  const int smem = smem_tiles > smem_merge ? smem_tiles : smem_merge;
  if (head_dim == 128) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(dec::attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); set = true; }
    cpi::launch_pdl(dec::attention_decode_kernel<128>, grid, dec::NT, smem, stream, p);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(dec::attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); set = true; }
    cpi::launch_pdl(dec::attention_decode_kernel<64>, grid, dec::NT, smem, stream, p);
  }
  if (check_launch("attention_decode")) return 2;
  if (n_splits > 1) {
    cpi::launch_pdl(dec::attention_combine_kernel, n_tokens * n_heads, head_dim <= 64 ? 64 : 128, 0, stream, 
        part_o, part_ml, (__nv_bfloat16*)out, n_splits, head_dim);
    return check_launch("attention_combine");
  }
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that may not allocate device memory (declared in
// attention_decode_noalloc.h; it has no counterpart in the reference).
//
// Same kernels as cpi_attention_decode, but the float32 partials of the key splits live in a fixed
// array inside this library instead of a buffer the caller allocates.  See the header for who needs
// this and for the rules of use.
namespace cpi {
namespace dec {

constexpr long kStaticScratchFloats = 2l << 20;             // 8 MiB per GPU that loads the library
static __device__ __align__(256) float g_split_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_scratch_ptr[kMaxDevices] = {};              // device address of the array, per device

// In host code `g_split_scratch` is only a handle for the runtime, not an address a kernel can use:
// ask the runtime for the array's device address once per device, with that device current.
static int static_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("attention_decode_noalloc: cannot identify the current device (%s)", cudaGetErrorString(e));
    return 1;
  }
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_split_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("attention_decode_noalloc: cudaGetSymbolAddress failed on device %d (%s)", dev, cudaGetErrorString(e));
      return 1;
    }
    g_scratch_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace dec
}  // namespace cpi

extern "C" long cpi_attention_decode_noalloc_capacity() { return cpi::dec::kStaticScratchFloats; }

extern "C" int cpi_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                            const int* page_table, int max_blocks, int page_size,
                                            const int* token_seq, const int* token_pos, const int* seq_slot,
                                            int n_tokens, int n_heads, int n_kv_heads, int head_dim, int window_kind,
                                            int window_size, float scale, int n_splits, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(n_splits >= 1, "attention_decode_noalloc: n_splits must be >= 1, got %d", n_splits);
  const long need = (long)n_tokens * n_heads * n_splits * (head_dim + 2);
  CPI_REQUIRE(n_splits == 1 || need <= dec::kStaticScratchFloats,
              "attention_decode_noalloc: %d tokens x %d heads x %d splits need %ld floats of scratch; the built-in "
              "array holds %ld (use fewer splits, or the allocating entry point)",
              n_tokens, n_heads, n_splits, need, dec::kStaticScratchFloats);
  float* scratch = nullptr;
  if (dec::static_scratch(&scratch)) return 1;
  float* part_o = scratch;
  float* part_ml = scratch + (long)n_tokens * n_heads * n_splits * head_dim;
  return cpi_attention_decode(q, out, k_cache, v_cache, page_table, max_blocks, page_size, token_seq, token_pos,
                              seq_slot, n_tokens, n_heads, n_kv_heads, head_dim, window_kind, window_size, scale,
                              n_splits, part_o, part_ml, stream);
}
