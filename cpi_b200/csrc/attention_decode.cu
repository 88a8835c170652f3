// Decode attention in bfloat16: one new token per sequence against its paged cache, split over the keys.
//
// A block serves one (split, key/value head, sequence): the G query heads that share the key/value head
// form the rows of a 16-row MMA tile, so every key and value byte is read once per group and not once
// per head.  Keys and values arrive page by page: a (page, head) tile of 64 positions x D is contiguous
// in the cache, and one thread fetches it with the copy engine (cp.async.bulk.tensor boxes of 64 positions
// x 64 features with the 128-byte swizzle) into a ring of shared-memory stages, several pages ahead of the
// arithmetic; an mbarrier per stage says when its bytes have landed.  Each of the four warps owns 16 keys
// of the page and runs its own online softmax (scores S = Q K^T and the product P V on mma.sync m16n8k16 with
// float32 accumulators; a 5..16-row problem is below the 64-row minimum of tcgen05, and the kernel is
// bound by the cache bytes, not by the tensor pipe).  Warps, then splits, are merged with the usual
// (max, sum) rescaling; with one split the block writes the output itself, otherwise it writes
// float32 partials that a small second kernel combines.
//
// Reference: gqa_decode_kernel (src/kernels/kernels_attention_decode.cu:868-951) visits one key per
// iteration with three block barriers each; formulas as in src/engine/llama4_cpu_engine.cpp:195-250.
// Positions outside [window low, pos] are masked; in a page that holds such positions their value rows
// are overwritten with zeros in shared memory before use, so that stale page contents can never reach
// the result (0 x NaN would).  The waits on the copy engine are bounded: when one runs out the block
// raises the error word, skips its arithmetic, gives the copies in flight time to land and returns.
#include "common.cuh"
#include <cuda.h>

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
  int* error_flag;                                  // set to 1 when a wait on the copy engine ran out
};

constexpr uint32_t kSpinLimit = 1u << 24;
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

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

// Shared tile of PAGE rows x D bf16 as the copy engine's 128-byte swizzle leaves it: one box of 64 features
// (rows of 128 bytes) after the other, and within a box the 16-byte chunk c of row r at chunk c ^ (r & 7).
// `chunk` counts the row's 16-byte chunks 0 .. D/8 - 1; the result is in elements.
template <int D> __device__ __forceinline__ int tile_off(int row, int chunk) {
  return (chunk >> 3) * (PAGE * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
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

template <int D> struct Stages { static constexpr int N = D > 64 ? 3 : 4; };    // pages in flight per block

template <int D>
__global__ void __launch_bounds__(NT) attention_decode_kernel(const __grid_constant__ CUtensorMap map_k,
                                                              const __grid_constant__ CUtensorMap map_v, Params p) {
  constexpr int KS = D / 16;                // k-steps of Q K^T
  constexpr int NO = D / 8;                 // n-tiles of the output
  constexpr int STAGES = Stages<D>::N;
  constexpr int TILE = PAGE * D;            // elements of one (page, head) tile
  constexpr uint32_t STAGE_TX = 2u * TILE * 2u;       // bytes of a stage: keys and values
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES];
  __shared__ int abort_s;                   // set by the first thread whose wait ran out; the others then stop waiting
  // the swizzle is a function of the address: tiles start on 1024-byte boundaries
  uint8_t* smem_raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [STAGES][PAGE][D]
  __nv_bfloat16* v_s = k_s + STAGES * TILE;                                    // [STAGES][PAGE][D]

  const int split = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full_bar[s], 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  volatile int* aborted = &abort_s;
  // Positions, slots and the page table were put in place by copies that ended before this step's first kernel;
  // they, and every cache page but the one that holds the newest position, are not written by the kernel before
  // this one (the head rotation stores the newest position's key and value only).  So the first pages are asked for
  // BEFORE the wait on that kernel: a block's first page takes ~3 us to arrive, which now passes under its tail.
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

  // one thread asks the copy engine for the page of block `blk` into stage `st`
  auto load_tile = [&](int blk, int st) {
    const int row0 = (table[blk] * p.n_kv_heads + kvh) * PAGE;      // first row of the (page, head) tile
    mbar_expect_tx(&full_bar[st], STAGE_TX);
#pragma unroll
    for (int h = 0; h < D / 64; ++h) {
      tma_load_2d(k_s + st * TILE + h * (PAGE * 64), &map_k, &full_bar[st], h * 64, row0);
      tma_load_2d(v_s + st * TILE + h * (PAGE * 64), &map_v, &full_bar[st], h * 64, row0);
    }
  };
  int asked = 0;                                                     // (thread 0) stages asked for so far
  if (tid == 0)
    for (; asked < STAGES && b_begin + asked < b_end && b_begin + asked != b_hi; ++asked) load_tile(b_begin + asked, asked);
  pdl_wait();
  if (tid == 0)
    for (; asked < STAGES && b_begin + asked < b_end; ++asked) load_tile(b_begin + asked, asked);

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

  float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};
  float o[NO][4];
#pragma unroll
  for (int i = 0; i < NO; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  for (int blk = b_begin; blk < b_end; ++blk) {
    const int it = blk - b_begin, buf = it % STAGES;
    // every thread passes the barrier at the end of each round whether its wait held or not
    bool live = !*aborted;
    if (live && !mbar_wait(&full_bar[buf], (it / STAGES) & 1)) { *aborted = 1; live = false; }
    const bool ragged = blk * PAGE < lo || blk * PAGE + PAGE - 1 > pos;      // the page holds positions outside the window
    if (live) {
    const __nv_bfloat16* kt = k_s + buf * TILE;
    __nv_bfloat16* vt = v_s + buf * TILE;
    const int key0 = warp * 16;                       // this warp's 16 keys of the page
    if (ragged) {
      // this warp's value rows outside [lo, pos] become zeros (two lanes per row, D / 16 chunks each)
      const int row = key0 + (lane >> 1), kp = blk * PAGE + row;
      if (kp < lo || kp > pos) {
#pragma unroll
        for (int c = 0; c < D / 16; ++c)
          *reinterpret_cast<uint4*>(vt + tile_off<D>(row, (lane & 1) * (D / 16) + c)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }

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
    }
    // the zeros written above must be ordered before the copy engine writes this stage again
    if (ragged) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();                                  // every warp is done with the stage: it is asked for again
    if (tid == 0 && blk + STAGES < b_end && !*aborted) load_tile(blk + STAGES, buf);
  }
  __syncthreads();
  if (*aborted) {
    // a wait ran out: say so, give the copies in flight time to land before the shared memory is released
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    return;
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
namespace cpi { namespace tc {
int get_map_2d_bf16(const void* ptr, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMap* out);
} }

// Blocks of the kernel that share an SM (by their shared memory), for the caller's choice of `n_splits`.
extern "C" int cpi_attention_decode_blocks_per_sm(int head_dim) {
  const int stages = head_dim > 64 ? dec::Stages<128>::N : dec::Stages<64>::N;
  const int smem = stages * 2 * dec::PAGE * head_dim * 2 + 2048;
  int dev = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess) {
    cudaGetLastError();
    return 1;
  }
  const int n = per_sm / smem;
  return n < 1 ? 1 : n;
}

// `n_pages`: pages of the cache tensors k_cache, v_cache [n_pages, n_kv_heads, page_size, head_dim].
// `error_flag`: an int32 on the device that is set to 1 when a block's wait on the copy engine runs out (may be null).
extern "C" int cpi_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache, long n_pages,
                                    const int* page_table, int max_blocks, int page_size, const int* token_seq,
                                    const int* token_pos, const int* seq_slot, int n_tokens, int n_heads,
                                    int n_kv_heads, int head_dim, int window_kind, int window_size, float scale,
                                    int n_splits, float* part_o, float* part_ml, int* error_flag,
                                    cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  CPI_REQUIRE(cpi_attention_decode_supported(n_heads, n_kv_heads, head_dim, page_size),
              "attention_decode: unsupported shape (heads %d/%d, head size %d, page %d)", n_heads, n_kv_heads, head_dim, page_size);
  CPI_REQUIRE(window_kind == 0 || window_size > 0, "attention_decode: window kind %d needs a size > 0", window_kind);
  CPI_REQUIRE(n_splits >= 1 && n_splits <= dec::kMaxSplits && n_tokens <= 65535, "attention_decode: bad grid (%d splits of at most %d, %d tokens)", n_splits, dec::kMaxSplits, n_tokens);
  CPI_REQUIRE(n_splits == 1 || (part_o && part_ml), "attention_decode: split scratch is missing");
  CPI_REQUIRE(n_pages > 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
              "attention_decode: the cache must hold at least one page and be 16-byte aligned");
  dec::Params p{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                page_table, max_blocks, token_seq, token_pos, seq_slot, n_heads, n_kv_heads, window_kind, window_size,
                scale * 1.4426950408889634f, n_splits, part_o, part_ml, error_flag};
  // the cache as rows of head_dim features: a (page, head) tile is 64 consecutive rows
  CUtensorMap mk, mv;
  const uint64_t kv_rows = (uint64_t)n_pages * n_kv_heads * dec::PAGE;
  if (tc::get_map_2d_bf16(k_cache, (uint64_t)head_dim, kv_rows, (uint64_t)head_dim * 2, 64, dec::PAGE, &mk)) return 1;
  if (tc::get_map_2d_bf16(v_cache, (uint64_t)head_dim, kv_rows, (uint64_t)head_dim * 2, 64, dec::PAGE, &mv)) return 1;
  dim3 grid(n_splits, n_kv_heads, n_tokens);
  const int stages = head_dim == 128 ? dec::Stages<128>::N : dec::Stages<64>::N;
  const int smem_tiles = stages * 2 * dec::PAGE * head_dim * 2;
  const int smem_merge = (4 * 16 * head_dim + 128) * 4;
  const int smem = (smem_tiles > smem_merge ? smem_tiles : smem_merge) + 1024;
  if (head_dim == 128) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(dec::attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); set = true; }
    cpi::launch_pdl(dec::attention_decode_kernel<128>, grid, dec::NT, smem, stream, mk, mv, p);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(dec::attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); set = true; }
    cpi::launch_pdl(dec::attention_decode_kernel<64>, grid, dec::NT, smem, stream, mk, mv, p);
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
                                            long n_pages, const int* page_table, int max_blocks, int page_size,
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
  return cpi_attention_decode(q, out, k_cache, v_cache, n_pages, page_table, max_blocks, page_size, token_seq,
                              token_pos, seq_slot, n_tokens, n_heads, n_kv_heads, head_dim, window_kind, window_size,
                              scale, n_splits, part_o, part_ml, nullptr, stream);
}
