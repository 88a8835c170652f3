// bfloat16 matrix product on pairs of SMs:  out[t, n] = sum_k X[t, k] * W[n, k]  for many tokens (prefill).
//
// Two CTAs of a cluster share one 256 x BN tile through `tcgen05.mma.cta_group::2`: each CTA stages 128
// weight rows (the M operand) and HALF of the token rows (the N operand) in its own shared memory, the
// leader CTA issues one MMA that reads both halves, and each CTA ends up with its 128 output features
// for all BN tokens in its own tensor memory.  Per SM and k-step that is 16 KB of weights + 16 KB of
// tokens for a 128 x 256 x 64 product, two thirds of what a single-CTA tile of the same shape pulls
// through the L2 -- and the L2 is what bounds the single-CTA kernel (gemm_tc.cu) at these sizes.
//
// Synchronisation: TMA loads of both CTAs complete on the LEADER's full barrier (`cta_group::2` loads may
// signal the peer's barrier; no multicast load is used); the leader's `tcgen05.commit` with
// `multicast::cluster` frees the stage in both CTAs and, at the end, tells both that the accumulators
// are complete.  Every wait is bounded; a CTA that gives up raises the error flag and leaves.
// Epilogues as in gemm_tc.cu: STORE, ADD (float32 residual), SWIGLU, with groups (routed experts), a
// per-token scale and output row scatter; no split-K here.
// The reference has no tensor-core kernel of its own (src/kernels/kernels_ops_matvec.cu:343-418 are
// SIMT GEMVs); this file has no counterpart there.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <cuda.h>

namespace cpi {
namespace tc {
int get_map_2d_bf16(const void* ptr, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMap* out);
int get_map_3d_bf16(const void* ptr, uint64_t inner, uint64_t rows, uint64_t groups, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMap* out);
}
namespace tc2 {

constexpr int BM = 128;          // output features per CTA (256 per pair)
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr uint32_t kSpinLimit = 1u << 24;
constexpr int kMaxSlots = 512;     // token tiles of a grouped product that the persistent kernel lists
enum Mode : int { kStore = 0, kAdd = 1, kSwiglu = 2 };

struct Params {
  void* out; long ldo;
  const int* out_rows;
  const float* row_scale;
  const int* group_offsets; int n_groups;      // routed experts: tokens [offsets[g], offsets[g+1]) use W[g]
  int T, bn, N, k_tiles;
  int* error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// loads of a CTA pair: data into this CTA's shared memory, completion on the barrier at cluster address `bar`
__device__ __forceinline__ void tma2_load_2d(void* smem, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(smem)), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(smem)), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// arrives on the barrier at the same shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint32_t instr_desc_pair(int n) {       // M = 256 over the pair
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
template <typename TO> __device__ __forceinline__ void store_out(TO* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int BN, int MODE, typename TO, int STAGES>
__global__ void __launch_bounds__(128) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                           const __grid_constant__ CUtensorMap map_x, Params p) {
  constexpr int ACC = MODE == kSwiglu ? 2 : 1;
  constexpr int HALF = BN / 2;                                   // token rows this CTA stages, at most
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = HALF * BK * 2;
  constexpr uint32_t STAGE_BYTES = ACC * A_BYTES + B_BYTES;
  constexpr int BOX_ROWS = 64;
  constexpr uint32_t BOX_BYTES = BOX_ROWS * BK * 2;
  constexpr uint32_t TMEM_COLS = ACC * BN;
  static_assert(BN % 128 == 0 && TMEM_COLS <= 512, "pair tiles are 128 or 256 tokens wide");
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int offs_s[257], tiles_s[256], found_s[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t rank = cluster_rank();                          // 0: leader (issues the MMAs), 1: peer
  pdl_launch_dependents();

  // ---- which tile (both CTAs of a pair share blockIdx.y, so they find the same one) ----
  int group = 0, t_begin = 0, t_end = p.T, tile_t = blockIdx.y;
  if (p.group_offsets) {
    pdl_wait();
    for (int g = tid; g < p.n_groups; g += 128) {
      const int b = p.group_offsets[g], e = p.group_offsets[g + 1];
      offs_s[g] = b;
      tiles_s[g] = (e - b + p.bn - 1) / p.bn;
      if (g == p.n_groups - 1) offs_s[g + 1] = e;
    }
    __syncthreads();
    if (tid == 0) {
      int rest = tile_t, hit = -1;
      for (int g = 0; g < p.n_groups; ++g) {
        if (rest < tiles_s[g]) { hit = g; break; }
        rest -= tiles_s[g];
      }
      found_s[0] = hit;
      found_s[1] = rest;
    }
    __syncthreads();
    if (found_s[0] < 0) return;                                  // both CTAs of the pair leave together
    group = found_s[0]; tile_t = found_s[1]; t_begin = offs_s[group]; t_end = offs_s[group + 1];
  }
  int pair_n = blockIdx.x >> 1;                                  // which 256 output features
  if (!p.group_offsets) {
    // Dense product: pairs are handed out (x fastest, then y) so that the ones running at the same time
    // cover a band of up to 8 token tiles times as many weight tiles as fit: a wave then pulls about
    // 8 + 9 operand strips through the L2 instead of 28 + 3, and the weights come from DRAM once.
    const int n_pairs = gridDim.x >> 1, n_tok = gridDim.y, W = 8;
    const int pid = blockIdx.y * n_pairs + pair_n;
    const int band = pid / (W * n_pairs), rem = pid - band * W * n_pairs;
    const int w_eff = min(W, n_tok - band * W);
    tile_t = band * W + rem % w_eff;
    pair_n = rem / w_eff;
  }
  const int n0 = (pair_n * 2 + (int)rank) * BM;                  // this CTA's output features
  const int t0 = t_begin + tile_t * p.bn;
  const int n_valid_t = min(p.bn, t_end - t0);
  const int n_mma = min(BN, (n_valid_t + 31) & ~31);             // MMA width: both halves stay multiples of 16
  const int half = n_mma / 2;                                    // token rows of the tile staged by each CTA
  const int n_boxes = (half + BOX_ROWS - 1) / BOX_ROWS;
  const uint32_t cta_tx = ACC * A_BYTES + (uint32_t)n_boxes * BOX_BYTES;
  const int n_kt = p.k_tiles;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();                                                // the peer's barriers exist before anyone signals them
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer (both CTAs): weights before the wait on the preceding kernel, tokens after ----
    const int n_early = p.group_offsets ? 0 : min(n_kt, STAGES);
    for (int i = 0; i < n_early; ++i) {
      uint8_t* st = smem + (size_t)i * STAGE_BYTES;
      const uint32_t bar = map_to_cta(smem_u32(&full_bar[i]), 0);
      if (rank == 0) mbar_expect_tx(&full_bar[i], 2 * cta_tx);
      tma2_load_3d(st, &map_w, bar, i * BK, n0, group);
      if (ACC == 2) tma2_load_3d(st + A_BYTES, &map_w, bar, i * BK, p.N + n0, group);
    }
    pdl_wait();
    for (int i = 0; i < n_early; ++i) {
      const uint32_t bar = map_to_cta(smem_u32(&full_bar[i]), 0);
      for (int b = 0; b < n_boxes; ++b)
        tma2_load_2d(smem + (size_t)i * STAGE_BYTES + ACC * A_BYTES + b * BOX_BYTES, &map_x, bar, i * BK,
                     t0 + (int)rank * half + b * BOX_ROWS);
    }
    for (int i = n_early; i < n_kt; ++i) {
      const int s = i % STAGES;
      if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abort_flag)) break;
      uint8_t* st = smem + (size_t)s * STAGE_BYTES;
      const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
      if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * cta_tx);
      tma2_load_3d(st, &map_w, bar, i * BK, n0, group);
      if (ACC == 2) tma2_load_3d(st + A_BYTES, &map_w, bar, i * BK, p.N + n0, group);
      for (int b = 0; b < n_boxes; ++b)
        tma2_load_2d(st + ACC * A_BYTES + b * BOX_BYTES, &map_x, bar, i * BK, t0 + (int)rank * half + b * BOX_ROWS);
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---- MMA issuer (leader only): one instruction spans both CTAs ----
    const uint32_t idesc = instr_desc_pair(n_mma);
    bool ok = true;
    for (int i = 0; i < n_kt && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(&full_bar[s], (i / STAGES) & 1, abort_flag);
      if (!ok) break;
      fence_after_sync();
      const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
      const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + ACC * A_BYTES);
#pragma unroll
      for (int j = 0; j < BK / UMMA_K; ++j) {
        const uint32_t acc = (i > 0 || j > 0) ? 1u : 0u;
        umma2_bf16(tmem_base, da + 2 * j, db + 2 * j, idesc, acc);
        if (ACC == 2) umma2_bf16(tmem_base + BN, smem_desc_sw128(a_addr + A_BYTES) + 2 * j, db + 2 * j, idesc, acc);
      }
      umma2_commit_both(&empty_bar[s]);
    }
    if (ok) umma2_commit_both(&accum_bar);
  }
  __syncwarp();

  // ---- epilogue: each CTA stores its 128 features of all the tile's tokens ----
  pdl_wait();
  bool ok = mbar_wait(&accum_bar, 0, abort_flag);
  fence_after_sync();
  ok = __syncthreads_and(ok && !abort_s) != 0;                   // one decision for the CTA
  const int row = warp * 32 + lane;
  const int n = n0 + row;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
  const int n_cols = min(BN, (n_valid_t + 15) & ~15);
  TO* out = reinterpret_cast<TO*>(p.out);
  const bool row_ok = n < p.N;
  if (ok && epi::staged_ok<TO>(p.out, p.ldo, n_valid_t)) {
    // the tile is turned in shared memory (the stages are idle: every MMA has completed) and leaves in
    // whole rows
    constexpr int kFit = (int)((size_t)STAGES * STAGE_BYTES / (128 * sizeof(TO))) / 16 * 16;   // columns the idle stages hold
      constexpr int kStageCols = kFit < BN ? kFit : BN;
      auto ld = [&](int c, float* d) { tmem_ld16(lane_addr + c, d); };
    auto ldu = [&](int c, float* d) { tmem_ld16(lane_addr + BN + c, d); };
    epi::staged<MODE, TO, kStageCols>(smem, ld, ldu, warp, lane, n0, p.N, t0, n_valid_t, n_cols, out, p.ldo, p.out_rows, p.row_scale);
  } else if (ok && MODE == kAdd) {
    float* outf = reinterpret_cast<float*>(p.out);
    float old[2][16];
    auto fetch = [&](int c, float* dst) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int col = c + j;
        dst[j] = (row_ok && col < n_valid_t) ? outf[(size_t)(p.out_rows ? p.out_rows[t0 + col] : t0 + col) * p.ldo + n] : 0.f;
      }
    };
    fetch(0, old[0]);
#pragma unroll 1
    for (int c = 0; c < n_cols; c += 32) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int cc = c + 16 * h;
        if (cc >= n_cols) break;
        if (cc + 16 < n_cols) fetch(cc + 16, old[h ^ 1]);
        float v[16];
        tmem_ld16(lane_addr + cc, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int col = cc + j;
          if (row_ok && col < n_valid_t) {
            const float s = p.row_scale ? p.row_scale[t0 + col] : 1.0f;
            outf[(size_t)(p.out_rows ? p.out_rows[t0 + col] : t0 + col) * p.ldo + n] = old[h][j] + v[j] * s;
          }
        }
      }
    }
  } else if (ok) {
#pragma unroll 1
    for (int c = 0; c < n_cols; c += 16) {
      float v[16], u[16];
      tmem_ld16(lane_addr + c, v);
      if (ACC == 2) tmem_ld16(lane_addr + BN + c, u);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int col = c + j;
        if (!row_ok || col >= n_valid_t) continue;
        const float s = p.row_scale ? p.row_scale[t0 + col] : 1.0f;
        float x = v[j] * s;
        if (MODE == kSwiglu) x = epi::silu_mul(x, u[j] * s);
        store_out<TO>(out + (size_t)(p.out_rows ? p.out_rows[t0 + col] : t0 + col) * p.ldo + n, x);
      }
    }
  }
  if (!ok) {
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 3);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();                                                // neither CTA leaves while the other may still use it
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
}

// ---------------------------------------------------------------------------------------------- persistent
// The same product with one pair per SM pair that works through a list of tiles (dense products only).
// Six warps per CTA: 0-3 own the accumulator's lanes and run the epilogue, warp 4 issues the TMA loads,
// warp 5 (of the leading CTA) the MMAs.  The stage ring runs on across tiles, and with one accumulator per
// tile there are two accumulator buffers in tensor memory: the MMAs of tile j+1 run while tile j is turned
// in shared memory and written out, so an SM pair's tiles follow each other at the tensor pipe's rate
// instead of each paying fill, drain and epilogue.  (With two accumulators, SwiGLU, the tensor memory
// holds one tile: its MMAs wait for the epilogue, but its loads do not.)
//   full[s] / empty[s]            stage ring, as above
//   acc_full[b]                   MMA -> epilogue warps of both CTAs (commit with multicast)
//   acc_empty[b] (in the leader)  epilogue warps of both CTAs -> MMA: one arrival per warp, 8 in all
template <int BN, int MODE, typename TO, int STAGES>
__global__ void __launch_bounds__(192) gemm_tc_pair_persistent_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                      const __grid_constant__ CUtensorMap map_x,
                                                                      Params p, int n_pairs, int n_tok) {
  constexpr int ACC = MODE == kSwiglu ? 2 : 1;
  constexpr int NB = ACC == 1 ? 2 : 1;                           // accumulator buffers in tensor memory
  constexpr int HALF = BN / 2;
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = HALF * BK * 2;
  constexpr uint32_t STAGE_BYTES = ACC * A_BYTES + B_BYTES;
  constexpr int BOX_ROWS = 64;
  constexpr uint32_t BOX_BYTES = BOX_ROWS * BK * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int EPI_COLS = 64;                                   // columns turned at a time
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[NB], acc_empty[NB];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s, n_live_s;
  __shared__ int slot_group[kMaxSlots], slot_t0[kMaxSlots], slot_rows[kMaxSlots];     // groups: the token tiles that hold rows
  __shared__ short slot_first[kMaxSlots], slot_count[kMaxSlots];                     // ... and their group's first tile and tile count

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* ring = smem;
  uint8_t* epi = smem + (size_t)STAGES * STAGE_BYTES;
  const uint32_t rank = cluster_rank();
  pdl_launch_dependents();
  const bool grouped = p.group_offsets != nullptr;
  if (grouped) {
    // the row lists come from the kernel before this one; one thread walks the groups and lists their tiles
    pdl_wait();
    if (tid == 0) {
      int n = 0;
      for (int g = 0; g < p.n_groups; ++g) {
        const int b = p.group_offsets[g], e = p.group_offsets[g + 1], first = n;
        // a group with more rows than a tile takes is cut into tiles of about equal size (a multiple of 32 rows):
        // the tile numbers go round the SM pairs, and a full tile beside a nearly empty one would give every
        // second pair the full ones
        const int count = (e - b + p.bn - 1) / p.bn;
        const int per = count > 0 ? (((e - b + count - 1) / count + 31) & ~31) : p.bn;
        for (int t = b; t < e && n < kMaxSlots; t += per) { slot_group[n] = g; slot_t0[n] = t; slot_rows[n] = min(per, e - t); ++n; }
        for (int i = first; i < n; ++i) { slot_first[i] = (short)first; slot_count[i] = (short)(n - first); }
      }
      n_live_s = n;
    }
    __syncthreads();
  }
  const int n_tok_live = grouped ? n_live_s : n_tok;
  const int n_tiles = n_pairs * n_tok_live;
  const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;
  const int n_kt = p.k_tiles;
  // tile number -> (first token row, rows, weight pair, group).  Dense: bands of 8 token tiles as in the kernel
  // above.  Groups: group after group, within a group weight pair after weight pair, and the group's token tiles
  // for one weight pair next to each other: the SM pairs that run them at the same time share the weights' way
  // through the L2, so a group's weights are read from memory once however many token tiles it has, and its rows
  // (a few MB) stay in the L2 while its weight pairs go by.
  auto tile_of = [&](int pid, int& t0, int& n_valid_t, int& pair_n, int& group) {
    if (grouped) {
      const int s = pid / n_pairs;                       // a tile of the group (its tiles own n_pairs numbers each)
      const int first = slot_first[s], count = slot_count[s];
      const int local = pid - first * n_pairs;
      pair_n = local / count;
      const int slot = first + (local - pair_n * count);
      group = slot_group[slot]; t0 = slot_t0[slot]; n_valid_t = slot_rows[slot];
      return;
    }
    const int W = 8;
    const int band = pid / (W * n_pairs), rem = pid - band * W * n_pairs;
    const int w_eff = min(W, n_tok - band * W);
    const int tile_t = band * W + rem % w_eff;
    pair_n = rem / w_eff;
    group = 0; t0 = tile_t * p.bn; n_valid_t = min(p.bn, p.T - t0);
  };

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < NB; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;

  if (warp == 4) {
    if (lane == 0) {
      // ---- TMA producer (both CTAs); weights need no wait on the preceding kernel, tokens do ----
      bool waited = false;
      int it = 0;
      for (int pid = cluster_id; pid < n_tiles; pid += n_clusters) {
        int t0, n_valid_t, pair_n, group;
        tile_of(pid, t0, n_valid_t, pair_n, group);
        const int n0 = (pair_n * 2 + (int)rank) * BM;
        const int half = min(BN, (n_valid_t + 31) & ~31) / 2;
        const int n_boxes = (half + BOX_ROWS - 1) / BOX_ROWS;
        const uint32_t cta_tx = ACC * A_BYTES + (uint32_t)n_boxes * BOX_BYTES;
        bool ok = true;
        for (int kt = 0; kt < n_kt; ++kt, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1, abort_flag)) { ok = false; break; }
          uint8_t* st = ring + (size_t)s * STAGE_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * cta_tx);
          tma2_load_3d(st, &map_w, bar, kt * BK, n0, group);
          if (ACC == 2) tma2_load_3d(st + A_BYTES, &map_w, bar, kt * BK, p.N + n0, group);
          if (!waited) { pdl_wait(); waited = true; }
          for (int b = 0; b < n_boxes; ++b)
            tma2_load_2d(st + ACC * A_BYTES + b * BOX_BYTES, &map_x, bar, kt * BK, t0 + (int)rank * half + b * BOX_ROWS);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && rank == 0) {
      // ---- MMA issuer (leader only) ----
      int it = 0, j = 0;
      bool ok = true;
      for (int pid = cluster_id; pid < n_tiles && ok; pid += n_clusters, ++j) {
        int t0, n_valid_t, pair_n, group;
        tile_of(pid, t0, n_valid_t, pair_n, group);
        const uint32_t idesc = instr_desc_pair(min(BN, (n_valid_t + 31) & ~31));
        const int b = j % NB;
        if (j >= NB) ok = mbar_wait(&acc_empty[b], ((j / NB) - 1) & 1, abort_flag);     // the epilogue has read it
        if (!ok) break;
        fence_after_sync();
        const uint32_t d0 = tmem_base + b * (ACC * BN);
        for (int kt = 0; kt < n_kt; ++kt, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, abort_flag);
          if (!ok) break;
          fence_after_sync();
          const uint32_t a_addr = smem_u32(ring + (size_t)s * STAGE_BYTES);
          const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + ACC * A_BYTES);
          const uint64_t da2 = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int q = 0; q < BK / UMMA_K; ++q) {
            const uint32_t acc = (kt > 0 || q > 0) ? 1u : 0u;
            umma2_bf16(d0, da + 2 * q, db + 2 * q, idesc, acc);
            if (ACC == 2) umma2_bf16(d0 + BN, da2 + 2 * q, db + 2 * q, idesc, acc);
          }
          umma2_commit_both(&empty_bar[s]);
        }
        if (ok) umma2_commit_both(&acc_full[b]);
      }
    }
  } else {
    // ---- epilogue: warps 0-3 of both CTAs; each CTA stores its 128 features of the tile's tokens ----
    pdl_wait();
    const uint32_t leader_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
    int j = 0;
    for (int pid = cluster_id; pid < n_tiles; pid += n_clusters, ++j) {
      int t0, n_valid_t, pair_n, group;
      tile_of(pid, t0, n_valid_t, pair_n, group);
      const int n0 = (pair_n * 2 + (int)rank) * BM;
      const int n_cols = min(BN, (n_valid_t + 15) & ~15);
      const int b = j % NB;
      mbar_wait(&acc_full[b], (j / NB) & 1, abort_flag);
      // one decision for the four warps (a named barrier has no time limit: nobody may leave alone); it also
      // keeps the turning buffer of the tile before from being overwritten while a warp still copies it out
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (abort_s) break;
      fence_after_sync();
      const uint32_t lane_addr = tmem_base + b * (ACC * BN) + ((uint32_t)(warp * 32) << 16);
      auto ld = [&](int c, float* d) { tmem_ld16(lane_addr + c, d); };
      auto ldu = [&](int c, float* d) { tmem_ld16(lane_addr + BN + c, d); };
      TO* out = reinterpret_cast<TO*>(p.out);
      epi::staged<MODE, TO, EPI_COLS>(epi, ld, ldu, warp, lane, n0, p.N, t0, n_valid_t, n_cols, out, p.ldo, p.out_rows,
                                      p.row_scale, epi::NamedSync<1, 128>());
      // the accumulator has been read (the last tensor-memory load of the tile precedes the last barrier above)
      fence_before_sync();
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];"
                     ::"r"(leader_empty0 + (uint32_t)(b * sizeof(uint64_t))) : "memory");
    }
  }
  __syncwarp();
  if (abort_s) {
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 4);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync();                                                // neither CTA leaves while the other may still use it
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
}

template <int BN, int MODE, typename TO>
static int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, int n_pairs, int n_tok,
                             cudaStream_t stream) {
  constexpr int ACC = MODE == kSwiglu ? 2 : 1;
  constexpr int STAGE = ACC * BM * BK * 2 + (BN / 2) * BK * 2;
  constexpr int EPI = 64 * 128 * (int)sizeof(TO);
  constexpr int S0 = (222 * 1024 - EPI) / STAGE;
  constexpr int STAGES = S0 > 8 ? 8 : S0;
  constexpr int SMEM = STAGES * STAGE + EPI;
  auto kern = gemm_tc_pair_persistent_kernel<BN, MODE, TO, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      set_error("gemm_tc_pair: cannot reserve %d bytes of shared memory", SMEM);
      return 1;
    }
    attr_set = true;
  }
  int dev = 0, n_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
  int clusters = n_sm / 2;
  if (clusters > n_pairs * n_tok) clusters = n_pairs * n_tok;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  count_launch();
  cudaLaunchKernelEx(&cfg, kern, mw, mx, p, n_pairs, n_tok);
  return check_launch("gemm_tc_pair_persistent");
}

template <int BN, int MODE, typename TO>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, cudaStream_t stream) {
  constexpr int ACC = MODE == kSwiglu ? 2 : 1;
  constexpr int STAGE = ACC * BM * BK * 2 + (BN / 2) * BK * 2;
  // One accumulator: half the shared memory per pair, so that two pairs share an SM pair and the epilogue
  // of one runs under the matrix product of the other (measured 1.4x).  Two accumulators fill the tensor
  // memory: one pair per SM pair, with all the stages.
  constexpr int SMEM_LIMIT = ACC == 1 ? 108 * 1024 : 196 * 1024;
  constexpr int S0 = SMEM_LIMIT / STAGE;
  constexpr int STAGES = S0 > 8 ? 8 : S0;
  constexpr int SMEM = STAGES * STAGE + 1024;
  auto kern = gemm_tc_pair_kernel<BN, MODE, TO, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      set_error("gemm_tc_pair: cannot reserve %d bytes of shared memory", SMEM);
      return 1;
    }
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  count_launch();
  cudaLaunchKernelEx(&cfg, kern, mw, mx, p);
  return check_launch("gemm_tc_pair");
}

}  // namespace tc2
}  // namespace cpi

using namespace cpi;

// Whether the paired kernel takes this product, and the token-tile width it would use (0: not taken).
// Dense products: one pair per SM pair working through a tile list (2: always), one launch slot per tile
// (0: always), or whichever measured faster (1, the default).  Both run at what the L2 can deliver to the
// SMs (a 256 x 256 pair tile at the tensor pipe's full rate would pull 64 bytes per cycle and SM, ~15 TB/s
// over the GPU; measured: the MMA thread of the persistent kernel waits for operands a third of the time).
// Two pairs sharing an SM pair hide that latency better for one accumulator; the persistent kernel wins
// where the epilogue is long or cannot overlap otherwise: SwiGLU (two accumulators fill the tensor memory,
// no second pair fits) and the read-modify-write of ADD at many tokens.
static int g_persistent = 1;
extern "C" void cpi_gemm_tc_pair_persistent(int mode) { g_persistent = mode; }

extern "C" int cpi_gemm_tc_pair_plan(int T, int N, int K, int swiglu, int n_groups) {
  if (N % 256 != 0 || K % 8 != 0) return 0;
  if (n_groups > 0) {
    // experts: one token tile per expert (its weights are then read once), sized for 1.5 x the mean rows
    if (n_groups > 256 || T < 64 * n_groups) return 0;
    const int want = (3 * ((T + n_groups - 1) / n_groups) + 1) / 2;
    return want > 128 ? 256 : 128;
  }
  if (T < 512) return 0;
  // one pair per two SMs at a time: time ~ waves x (weight rows + half the tile width) per SM
  const long sm_pairs = cpi::sm_count() / 2 > 0 ? cpi::sm_count() / 2 : 1;
  long best_cost = -1;
  int bn = 0;
  const long pairs_x = N / 256;
  const int w_rows = swiglu ? 256 : 128;
  for (int cand = 256; cand >= 160; cand -= 32) {
    const long pairs = pairs_x * ((T + cand - 1) / cand);
    const long waves = (pairs + sm_pairs - 1) / sm_pairs;
    const long cost = waves * (w_rows + cand / 2 + 16);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; bn = cand; }
  }
  return bn;
}

// x [T, K] bf16 (row stride ldx), w [N or 2N][K] bf16 contiguous, out [T, N]; bn from cpi_gemm_tc_pair_plan.
extern "C" int cpi_gemm_tc_pair(const void* x, long ldx, const void* w, void* out, int out_dtype, long ldo,
                                const int* out_rows, const float* row_scale, const int* group_offsets, int n_groups,
                                int T, int N, int K, int mode, int bn, int* error_flag, cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  CPI_REQUIRE(N % 256 == 0 && K % 8 == 0 && ldx % 8 == 0, "gemm_tc_pair: N (%d) must be a multiple of 256, K (%d) and the row stride of 8", N, K);
  CPI_REQUIRE(bn >= 32 && bn <= 256 && bn % 32 == 0, "gemm_tc_pair: token tile %d (multiples of 32 up to 256)", bn);
  CPI_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0, "gemm_tc_pair: operands must be 16-byte aligned");
  CPI_REQUIRE(mode != tc2::kAdd || out_dtype == kF32, "gemm_tc_pair: ADD mode needs a float32 output");
  CPI_REQUIRE(mode != tc2::kSwiglu || out_dtype == kBF16, "gemm_tc_pair: SWIGLU mode writes bfloat16");
  const int acc = mode == tc2::kSwiglu ? 2 : 1;
  CUtensorMap mw, mx;
  CPI_REQUIRE(n_groups <= 256, "gemm_tc_pair: %d groups (at most 256)", n_groups);
  if (tc::get_map_3d_bf16(w, (uint64_t)K, (uint64_t)acc * N, (uint64_t)(n_groups > 0 ? n_groups : 1), tc2::BK, tc2::BM, &mw)) return 1;
  if (tc::get_map_2d_bf16(x, (uint64_t)K, (uint64_t)T, (uint64_t)ldx * 2, tc2::BK, 64, &mx)) return 1;
  tc2::Params p{out, ldo, out_rows, row_scale, group_offsets, n_groups, T, bn, N, (K + tc2::BK - 1) / tc2::BK, error_flag};
  dim3 grid(N / tc2::BM, (T + bn - 1) / bn + (n_groups > 0 ? (T < n_groups ? T : n_groups) : 0), 1);
  CPI_REQUIRE(grid.y <= 65535, "gemm_tc_pair: too many token tiles (%u)", grid.y);
  const int cap = bn <= 128 ? 128 : 256;
  // (ADD: the persistent kernel wins where the mainloop is short against the epilogue; measured at 8,192 tokens
  // with the copy engine's add: K = 5120 314 against 321 us, K = 8192 513 against 495 us)
  const bool persistent = g_persistent == 2 || (g_persistent == 1 && (mode == tc2::kSwiglu ||
                                                (mode == tc2::kAdd && T >= 4096 && K <= 6144)));
  const int n_slots = (T + bn - 1) / bn + (n_groups > 0 ? (T < n_groups ? T : n_groups) : 0);
  const bool persistent_groups = (g_persistent == 2 || (g_persistent == 1 && mode == tc2::kSwiglu)) && n_groups > 0 &&
                                 n_slots <= tc2::kMaxSlots;      // (measured: 2 % faster for SwiGLU, slower for STORE)
  if ((n_groups == 0 ? persistent : persistent_groups) && cap == 256) {
    const int n_pairs = N / 256, n_tok = n_slots;
    if (mode == tc2::kStore && out_dtype == kBF16) return tc2::launch_persistent<256, tc2::kStore, __nv_bfloat16>(mw, mx, p, n_pairs, n_tok, stream);
    if (mode == tc2::kStore && out_dtype == kF32) return tc2::launch_persistent<256, tc2::kStore, float>(mw, mx, p, n_pairs, n_tok, stream);
    if (mode == tc2::kAdd) return tc2::launch_persistent<256, tc2::kAdd, float>(mw, mx, p, n_pairs, n_tok, stream);
    if (mode == tc2::kSwiglu) return tc2::launch_persistent<256, tc2::kSwiglu, __nv_bfloat16>(mw, mx, p, n_pairs, n_tok, stream);
  }
#define CPI_PAIR(CAP)                                                                                         \
  if (mode == tc2::kStore && out_dtype == kBF16) return tc2::launch<CAP, tc2::kStore, __nv_bfloat16>(mw, mx, p, grid, stream); \
  if (mode == tc2::kStore && out_dtype == kF32) return tc2::launch<CAP, tc2::kStore, float>(mw, mx, p, grid, stream);         \
  if (mode == tc2::kAdd) return tc2::launch<CAP, tc2::kAdd, float>(mw, mx, p, grid, stream);                                  \
  if (mode == tc2::kSwiglu) return tc2::launch<CAP, tc2::kSwiglu, __nv_bfloat16>(mw, mx, p, grid, stream);
  if (cap == 128) { CPI_PAIR(128) } else { CPI_PAIR(256) }
#undef CPI_PAIR
  set_error("gemm_tc_pair: unsupported mode %d with output dtype %d", mode, out_dtype);
  return 1;
}
