// bfloat16 matrix product on the 5th-generation tensor cores:  out[t, n] = sum_k X[t, k] * W[g][n, k].
//
// One kernel for decode (a handful of tokens) and prefill (thousands).  The WEIGHT tile is the MMA's
// M operand (128 output features x 64 k), the TOKEN tile its N operand (16..256 tokens x 64 k); both
// are K-major, staged in shared memory by TMA with the 128-byte swizzle and consumed by
// tcgen05.mma (kind::f16, bf16 x bf16 -> fp32) with the accumulator in tensor memory.  A decode step
// therefore fills the 128-wide MMA with weight rows however few tokens there are, and streams every
// weight byte exactly once.  Roles inside a CTA of 128 threads: one elected thread of warp 0 issues
// TMA, one of warp 1 issues MMA; a ring of `stages` buffers with full/empty mbarriers couples them;
// after the last k-tile all four warps read their 32 accumulator lanes with tcgen05.ld and run the
// epilogue.  The reference has no tensor-core kernel of its own: its counterparts are SIMT GEMV
// kernels (src/kernels/kernels_ops_matvec.cu:343-418) and one cublasGemmEx call
// (src/engine/llama4_cuda_engine_setup.cu:579-605).
//
// Epilogues (same meaning as the FP32-pipe kernel):  STORE, ADD (float32 residual), SWIGLU (two
// accumulators: rows n and N + n of W; out = silu(g) * u).  Optional per-token scale, output row
// scatter, and groups (routed experts): tokens [offsets[g], offsets[g+1]) use W[g].
//
// Split-K: when a launch has too few tiles to fill the GPU, the k range is cut into `splits` parts (up
// to 8, token tiles up to 128), summed in split order (a fixed order: the result does not depend on
// arrival order).  The CTAs of a tile form a thread-block cluster along z.  Each puts its raw
// accumulators into its own shared memory; after a cluster barrier every CTA sums a share of the tile's
// columns over all CTAs' shared memory (distributed shared memory loads) and applies the epilogue to
// them.  No global scratch, and the merge runs in parallel.
//
// Every mbarrier wait is bounded (`spin_limit` polls): when it runs out the CTA raises `*error_flag`,
// stops issuing work, lets copies in flight land, frees its tensor memory and returns.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>

namespace cpi {
namespace tc {

constexpr int BM = 128;          // output features per tile (MMA M)
constexpr int BK = 64;           // k elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int UMMA_K = 16;
constexpr uint32_t kSpinLimit = 1u << 24;      // polls of one wait before a CTA gives up (launches may pass fewer)

enum Mode : int { kStore = 0, kAdd = 1, kSwiglu = 2 };

struct Params {
  void* out; long ldo;
  const int* out_rows;
  const float* row_scale;
  const int* group_offsets; int n_groups;
  int T;               // logical token rows (all groups)
  int bn;              // token rows per tile: a multiple of 16, at most the kernel's BN
  int N;               // output features
  int k_tiles;         // ceil(K / 64)
  int splits, k_tiles_per_split;   // splits > 1: the splits of a tile are one cluster along z
  int tiles_on_x;      // 1: blockIdx.x counts token tiles and blockIdx.y weight tiles (groups with many tokens)
  int* error_flag;
  uint32_t spin_limit; // polls of one barrier wait before the CTA gives up
  uint32_t tx_extra;   // bytes added to what a stage's barrier expects (0 but in the test of the give-up path)
};

// ---------------------------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
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
// Bounded wait: false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                          // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}
__host__ __device__ constexpr uint32_t instr_desc_bf16(int n) {
  return (1u << 4)                   // D format: F32
       | (1u << 7) | (1u << 10)      // A, B format: BF16
       | ((uint32_t)(n >> 3) << 17)  // N
       | ((uint32_t)(BM >> 4) << 24);  // M
}

template <typename TO> __device__ __forceinline__ void store_out(TO* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------------- kernel
template <int BN, int MODE, typename TO, int STAGES>
__global__ void __launch_bounds__(128) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                      const __grid_constant__ CUtensorMap map_x, Params p) {
  constexpr int ACC = MODE == kSwiglu ? 2 : 1;
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = ACC * A_BYTES + B_BYTES;
  constexpr int BOX_ROWS = BN < 64 ? BN : 64;           // token rows per TMA box of the activation tile
  constexpr uint32_t BOX_BYTES = BOX_ROWS * BK * 2;
  constexpr uint32_t TMEM_COLS = ACC * BN < 32 ? 32 : ACC * BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int offs_s[257], tiles_s[256], found_s[2];   // group offsets and tile counts (at most 256 groups)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  pdl_launch_dependents();
  // ---- which tile ----
  // Groups with many tokens: the token tiles of one (weight tile, group) are neighbours in launch order,
  // so the second one finds the weight strip in the L2 that the first one pulled from DRAM.
  int group = 0, t_begin = 0, t_end = p.T, tile_t = p.tiles_on_x ? blockIdx.x : blockIdx.y;
  if (p.group_offsets) {
    pdl_wait();                                  // the row lists come from the kernel before this one
    // One division per group, done by one thread each; thread 0 then walks the counts.  (Every CTA of the
    // launch does this, also the many that find no tile, so it has to be cheap.)
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
    const bool found = found_s[0] >= 0;
    if (found) { group = found_s[0]; tile_t = found_s[1]; t_begin = offs_s[group]; t_end = offs_s[group + 1]; }
    if (!found) return;
  }
  const int t0 = t_begin + tile_t * p.bn;
  if (t0 >= t_end) return;
  const int n0 = (p.tiles_on_x ? blockIdx.y : blockIdx.x) * BM;
  const int split = blockIdx.z;
  const int kt_begin = split * p.k_tiles_per_split;
  const int kt_end = min(p.k_tiles, kt_begin + p.k_tiles_per_split);
  const int n_kt = kt_end - kt_begin;
  // only the boxes that hold rows of this tile are fetched (a group's tail tile may hold few)
  const int n_boxes = (min(p.bn, t_end - t0) + BOX_ROWS - 1) / BOX_ROWS;
  const uint32_t stage_tx = ACC * A_BYTES + (uint32_t)n_boxes * BOX_BYTES + p.tx_extra;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accum_bar, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, TMEM_COLS);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort_flag = &abort_s;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ----
    // Weights are written by no kernel, so their tiles for the first stages are requested before the
    // wait on the preceding kernel; the activation tiles follow it.
    const int n_early = p.group_offsets ? 0 : min(n_kt, STAGES);
    for (int i = 0; i < n_early; ++i) {
      uint8_t* st = smem + (size_t)i * STAGE_BYTES;
      mbar_expect_tx(&full_bar[i], stage_tx);
      const int k = (kt_begin + i) * BK;
      tma_load_3d(st, &map_w, &full_bar[i], k, n0, group);
      if (ACC == 2) tma_load_3d(st + A_BYTES, &map_w, &full_bar[i], k, p.N + n0, group);
    }
    pdl_wait();
    for (int i = 0; i < n_early; ++i)
      for (int b = 0; b < n_boxes; ++b)
        tma_load_2d(smem + (size_t)i * STAGE_BYTES + ACC * A_BYTES + b * BOX_BYTES, &map_x, &full_bar[i],
                    (kt_begin + i) * BK, t0 + b * BOX_ROWS);
    for (int i = n_early; i < n_kt; ++i) {
      const int s = i % STAGES;
      if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abort_flag, p.spin_limit)) break;
      uint8_t* st = smem + (size_t)s * STAGE_BYTES;
      mbar_expect_tx(&full_bar[s], stage_tx);
      const int k = (kt_begin + i) * BK;
      tma_load_3d(st, &map_w, &full_bar[s], k, n0, group);
      if (ACC == 2) tma_load_3d(st + A_BYTES, &map_w, &full_bar[s], k, p.N + n0, group);
      for (int b = 0; b < n_boxes; ++b)
        tma_load_2d(st + ACC * A_BYTES + b * BOX_BYTES, &map_x, &full_bar[s], k, t0 + b * BOX_ROWS);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    // The MMA's N is a run-time field of the instruction descriptor: a tile with few rows (the tail of a
    // group, or a group with few tokens) multiplies only those columns, rounded up to 16.
    const int n_rows_here = min(p.bn, (p.group_offsets ? t_end : p.T) - t0);
    const uint32_t idesc = instr_desc_bf16(min(BN, (n_rows_here + 15) & ~15));
    bool ok = true;
    for (int i = 0; i < n_kt && ok; ++i) {
      const int s = i % STAGES;
      ok = mbar_wait(&full_bar[s], (i / STAGES) & 1, abort_flag, p.spin_limit);
      if (!ok) break;
      fence_after_sync();
      const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
      const uint64_t da = smem_desc_sw128(a_addr), db = smem_desc_sw128(a_addr + ACC * A_BYTES);
#pragma unroll
      for (int j = 0; j < BK / UMMA_K; ++j) {
        const uint32_t acc = (i > 0 || j > 0) ? 1u : 0u;
        umma_bf16(tmem_base, da + 2 * j, db + 2 * j, idesc, acc);
        if (ACC == 2) umma_bf16(tmem_base + BN, smem_desc_sw128(a_addr + A_BYTES) + 2 * j, db + 2 * j, idesc, acc);
      }
      umma_commit(&empty_bar[s]);       // frees the stage once these MMAs have read it
    }
    if (ok) umma_commit(&accum_bar);    // accumulators complete
  }
  __syncwarp();

  // ---- epilogue: all four warps ----
  pdl_wait();                                    // before any global read or write of this thread
  bool ok = mbar_wait(&accum_bar, 0, abort_flag, p.spin_limit);
  fence_after_sync();
  ok = __syncthreads_and(ok && !abort_s) != 0;            // one decision for the CTA

  const int row = warp * 32 + lane;                       // accumulator lane = output feature n0 + row
  const int n = n0 + row;
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
  const int n_valid_t = min(p.bn, t_end - t0);
  const int n_cols = min(BN, (n_valid_t + 15) & ~15);          // columns the MMAs wrote
  TO* out = reinterpret_cast<TO*>(p.out);

  auto emit = [&](int col, float v, float u) {
    const int lr = t0 + col;
    if (col >= n_valid_t || n >= p.N) return;
    const float s = p.row_scale ? p.row_scale[lr] : 1.0f;
    v *= s;
    TO* o = out + (size_t)(p.out_rows ? p.out_rows[lr] : lr) * p.ldo + n;
    if (MODE == kSwiglu) {
      u *= s;
      store_out<TO>(o, epi::silu_mul(v, u));
    } else if (MODE == kAdd) {
      store_out<TO>(o, to_f32(*o) + v);
    } else {
      store_out<TO>(o, v);
    }
  };

  if (p.splits == 1) {
    if (!ok) {
    } else if (epi::staged_ok<TO>(p.out, p.ldo, n_valid_t)) {
      // wide tile: turned in shared memory (the stages are idle: every MMA has completed), leaves in whole rows
      constexpr int kFit = (int)((size_t)STAGES * STAGE_BYTES / (128 * sizeof(TO))) / 16 * 16;   // columns the idle stages hold
      constexpr int kStageCols = kFit < BN ? kFit : BN;
      auto ld = [&](int c, float* d) { tmem_ld16(lane_addr + c, d); };
      auto ldu = [&](int c, float* d) { tmem_ld16(lane_addr + BN + c, d); };
      epi::staged<MODE, TO, kStageCols>(smem, ld, ldu, warp, lane, n0, p.N, t0, n_valid_t, n_cols, out, p.ldo, p.out_rows, p.row_scale);
    } else if (MODE == kAdd) {
      // read-modify-write of the residual: the old values of chunk c+1 are fetched while chunk c is added,
      // so that their latency hides behind the tensor-memory load
      const bool row_ok = n < p.N;
      float* outf = reinterpret_cast<float*>(p.out);
      float old[2][16];
      auto fetch = [&](int c, float* dst) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int col = c + j, lr = t0 + col;
          dst[j] = (row_ok && col < n_valid_t) ? outf[(size_t)(p.out_rows ? p.out_rows[lr] : lr) * p.ldo + n] : 0.f;
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
            const int col = cc + j, lr = t0 + col;
            if (row_ok && col < n_valid_t) {
              const float s = p.row_scale ? p.row_scale[lr] : 1.0f;
              outf[(size_t)(p.out_rows ? p.out_rows[lr] : lr) * p.ldo + n] = old[h][j] + v[j] * s;
            }
          }
        }
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < n_cols; c += 16) {
        float v[16], u[16];
        tmem_ld16(lane_addr + c, v);
        if (ACC == 2) tmem_ld16(lane_addr + BN + c, u);
#pragma unroll
        for (int j = 0; j < 16; ++j) emit(c + j, v[j], ACC == 2 ? u[j] : 0.f);
      }
    }
  } else {
    // Every thread of every CTA of the cluster passes both barriers, whether its own waits held or not.
    if constexpr (BN <= 128) {
      static_assert((size_t)ACC * BN * BM * 4 <= (size_t)STAGES * STAGE_BYTES, "the stages must hold a tile of floats");
      float* red = reinterpret_cast<float*>(smem);        // [acc][col][row]; the stages are idle by now
      if (ok) {
#pragma unroll 1
        for (int a = 0; a < ACC; ++a)
#pragma unroll 1
          for (int c = 0; c < n_cols; c += 16) {
            float v[16];
            tmem_ld16(lane_addr + a * BN + c, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) red[((size_t)a * BN + c + j) * BM + row] = v[j];
          }
      }
      cluster_sync();
      if (ok) {
        const int rank = (int)cluster_rank();
        const uint32_t mine = smem_u32(red + row);
        uint32_t peer[8];
#pragma unroll
        for (int z = 0; z < 8; ++z) peer[z] = map_to_cta(mine, z < p.splits ? z : 0);
        // this CTA's share: columns 4 rank .. 4 rank + 3, then every (4 splits)-th group of four
#pragma unroll 1
        for (int c0 = 4 * rank; c0 < n_valid_t; c0 += 4 * p.splits) {
          float sum[ACC][4];
#pragma unroll
          for (int a = 0; a < ACC; ++a) {
            float part[4][8];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int z = 0; z < 8; ++z)
                part[j][z] = (z < p.splits && c0 + j < n_valid_t)
                                 ? ld_cluster_f32(peer[z] + (uint32_t)(((size_t)a * BN + c0 + j) * BM * 4)) : 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float t = 0.f;
#pragma unroll
              for (int z = 0; z < 8; ++z) if (z < p.splits) t += part[j][z];
              sum[a][j] = t;
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) emit(c0 + j, sum[0][j], sum[ACC - 1][j]);
        }
      }
      cluster_sync();                                     // nobody leaves while its shared memory is being read
    }
  }

  if (!ok) {
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    // give copies in flight time to land before the shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

struct MapKey {
  const void* ptr; uint64_t d0, d1, d2, s1, s2; uint32_t b0, b1;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
    return h;
  }
};

// bf16 tensor [d2][d1][d0] with byte strides s1, s2; box b0 x b1 x 1, 128-byte swizzle.
static int get_map(const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2, uint32_t b0,
                   uint32_t b1, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.ptr = ptr; key.d0 = d0; key.d1 = d1; key.d2 = d2; key.s1 = s1; key.s2 = s2; key.b0 = b0; key.b1 = b1;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("gemm_tc: cuTensorMapEncodeTiled is not available from the driver"); return 1; }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = d2 > 0 ? 3 : 2;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r); return 1; }
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// 2-D bf16 tensor [rows][inner] with a row stride in bytes; box box_inner x box_rows (other kernels use it too)
int get_map_2d_bf16(const void* ptr, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMap* out) {
  return get_map(ptr, inner, rows, 0, row_stride_bytes, 0, box_inner, box_rows, out);
}

// 3-D bf16 tensor [groups][rows][inner], contiguous; box box_inner x box_rows x 1 (the paired kernel uses it too)
int get_map_3d_bf16(const void* ptr, uint64_t inner, uint64_t rows, uint64_t groups, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMap* out) {
  return get_map(ptr, inner, rows, groups, inner * 2, inner * 2 * rows, box_inner, box_rows, out);
}

template <int BN, int MODE, typename TO>
struct Variant {
  static constexpr int ACC = MODE == kSwiglu ? 2 : 1;
  static constexpr int STAGE = ACC * BM * BK * 2 + BN * BK * 2;
  // two CTAs per SM where the stages stay deep enough: one's epilogue then runs under the other's loads
  static constexpr int SMEM_LIMIT = (BN <= 32 || (BN == 64 && ACC == 1)) ? 108 * 1024 : 196 * 1024;
  static constexpr int S0 = SMEM_LIMIT / STAGE;
  static constexpr int STAGES = S0 > 8 ? 8 : (S0 < 2 ? 2 : S0);
  static constexpr int SMEM = STAGES * STAGE + 1024;
  using Kernel = void (*)(const CUtensorMap, const CUtensorMap, Params);
  static Kernel kernel() { return gemm_tc_kernel<BN, MODE, TO, STAGES>; }

  static bool prepare() {
    static bool done = false;
    if (!done) {
      if (cudaFuncSetAttribute(kernel(), cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
        set_error("gemm_tc: cannot reserve %d bytes of shared memory", SMEM);
        return false;
      }
      // all of the SM's configurable memory as shared memory: two CTAs of the narrow variants then fit
      cudaFuncSetAttribute(kernel(), cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
      cudaGetLastError();
      done = true;
    }
    return true;
  }

  // CTAs of this variant that share an SM.  Counted here from shared memory and tensor-memory columns:
  // the runtime's occupancy calculator answers 1 for every kernel that allocates tensor memory, although
  // such CTAs do run side by side (measured: 296 CTAs of 100 KB with tensor memory ran at once).
  static int blocks_per_sm() {
    static int n = -1;
    if (n < 0) {
      n = 1;
      cudaFuncAttributes fa;
      int dev = 0, per_sm = 0, reserved = 0;
      if (prepare() && cudaFuncGetAttributes(&fa, kernel()) == cudaSuccess && cudaGetDevice(&dev) == cudaSuccess &&
          cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess &&
          cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) == cudaSuccess) {
        const int by_smem = per_sm / (SMEM + (int)fa.sharedSizeBytes + reserved);
        const int cols = ACC * BN < 32 ? 32 : ACC * BN;
        const int by_tmem = 512 / cols;
        n = by_smem < by_tmem ? by_smem : by_tmem;
        if (n < 1) n = 1;
      } else {
        cudaGetLastError();
      }
    }
    return n;
  }

  // Clusters of `size` CTAs along z that the GPU holds at once (0 when it cannot say): the runtime's count
  // (which knows how SMs group into GPCs, and assumes one CTA per SM) times the CTAs that share an SM.
  static int max_clusters(int size) {
    static int cache[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
    if (size < 1 || size > 8) return 0;
    if (cache[size] < 0) {
      cache[size] = 0;
      if (prepare()) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, size);
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = SMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)size;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel(), &cfg) == cudaSuccess && n > 0) cache[size] = n * blocks_per_sm();
        else cudaGetLastError();
      }
    }
    return cache[size];
  }

  static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, cudaStream_t stream) {
    if (!prepare()) return 1;
    if (p.splits > 1) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(128);
      cfg.dynamicSmemBytes = SMEM;
      cfg.stream = stream;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)p.splits;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      count_launch();
      cudaLaunchKernelEx(&cfg, kernel(), mw, mx, p);
    } else {
      cpi::launch_pdl(kernel(), grid, 128, SMEM, stream, mw, mx, p);
    }
    return check_launch("gemm_tc");
  }
};

// Clusters of `size` that fit at once for the kernel variant of a token tile and epilogue.
static int max_clusters_for(int bn_cap, bool swiglu, int size) {
  switch (bn_cap) {
    case 16:  return swiglu ? Variant<16, kSwiglu, __nv_bfloat16>::max_clusters(size) : Variant<16, kStore, __nv_bfloat16>::max_clusters(size);
    case 32:  return swiglu ? Variant<32, kSwiglu, __nv_bfloat16>::max_clusters(size) : Variant<32, kStore, __nv_bfloat16>::max_clusters(size);
    case 64:  return swiglu ? Variant<64, kSwiglu, __nv_bfloat16>::max_clusters(size) : Variant<64, kStore, __nv_bfloat16>::max_clusters(size);
    case 128: return swiglu ? Variant<128, kSwiglu, __nv_bfloat16>::max_clusters(size) : Variant<128, kStore, __nv_bfloat16>::max_clusters(size);
  }
  return 0;
}

template <int MODE, typename TO>
static int launch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, cudaStream_t s) {
  switch (bn) {
    case 16:  return Variant<16, MODE, TO>::launch(mw, mx, p, grid, s);
    case 32:  return Variant<32, MODE, TO>::launch(mw, mx, p, grid, s);
    case 64:  return Variant<64, MODE, TO>::launch(mw, mx, p, grid, s);
    case 128: return Variant<128, MODE, TO>::launch(mw, mx, p, grid, s);
    case 256: return Variant<256, MODE, TO>::launch(mw, mx, p, grid, s);
  }
  set_error("gemm_tc: token tile %d is not supported", bn);
  return 1;
}

}  // namespace tc
}  // namespace cpi

using namespace cpi;

// Polls of one barrier wait before a CTA gives up, and bytes added to what each stage's barrier expects.  The
// defaults are those of every ordinary launch; the test of the give-up path sets a short limit and a byte count
// that the stage's loads do not reach, launches once, and sets them back.
static uint32_t g_spin_limit = tc::kSpinLimit, g_tx_extra = 0;
extern "C" void cpi_gemm_tc_wait_probe(int spin_limit, int tx_extra) {
  g_spin_limit = spin_limit > 0 ? (uint32_t)spin_limit : tc::kSpinLimit;
  g_tx_extra = tx_extra > 0 ? (uint32_t)tx_extra : 0;
}

// Token-tile width and split count for a launch (also used by the caller to size the scratch).
// tiles_hint = expected token tiles per group (rows per group / bn, rounded up), groups_hint = groups in use.
extern "C" int cpi_gemm_tc_plan(int T, int N, int K, int n_groups, int swiglu, int* bn_out, int* splits_out,
                                int* live_y_out) {
  // groups: rows are spread unevenly, and a group that needs a second token tile reads its weights twice;
  // size the tile for one and a half times the mean
  const int rows_per_group = n_groups > 0 ? (3 * ((T + n_groups - 1) / n_groups) + 1) / 2 : T;
  int bn = 16;
  while (bn < 256 && bn < rows_per_group) bn *= 2;
  if (swiglu && bn > 256) bn = 256;
  const int n_tiles = (N + tc::BM - 1) / tc::BM;
  const long sms = sm_count();
  if (n_groups == 0 && T > 256) {
    // many tokens: one CTA per SM at a time, and a tile's time follows the operand bytes it pulls through
    // the L2 per k-step (128 or 256 weight rows + the token rows), so time ~ waves x (weight rows + width);
    // a somewhat narrower tile can turn "3.03 waves" into 3
    long best_cost = -1;
    const int w_rows = swiglu ? 256 : 128;
    for (int cand = 256; cand >= 128; cand -= 16) {
      const long ctas = (long)n_tiles * ((T + cand - 1) / cand);
      const long waves = (ctas + sms - 1) / sms;
      const long cost = waves * (cand + w_rows);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; bn = cand; }
    }
  }
  // token tiles that can hold rows: sum_g ceil(rows_g / bn) <= ceil(T / bn) + min(T, groups); they are
  // the first values of blockIdx.y, so scratch is only needed for those
  const int live_y = (T + bn - 1) / bn + (n_groups > 0 ? (T < n_groups ? T : n_groups) : 0);
  const int k_tiles = (K + tc::BK - 1) / tc::BK;
  int splits = 1;
  // CTAs that will really run: one per token tile; with groups at most one more per group that has rows
  const int run_y = n_groups > 0 ? (T <= n_groups ? T : (T + bn - 1) / bn + n_groups / 2) : (T + bn - 1) / bn;
  const long ctas = (long)n_tiles * (run_y > 0 ? run_y : 1);
  const int max_by_k = k_tiles / 4 > 0 ? k_tiles / 4 : 1;     // at least 4 k-tiles per split
  if (bn <= 128 && (bn & (bn - 1)) == 0) {
    // the splits of a tile are a cluster: the most splits (up to 8) whose clusters are all resident at
    // once, so that the launch is one wave (a launch of 1.1 waves takes as long as one of 2)
    for (int s = max_by_k < 8 ? max_by_k : 8; s >= 2; --s) {
      const int per_s = (k_tiles + s - 1) / s;
      if ((long)(s - 1) * per_s >= k_tiles) continue;           // would leave an empty split
      if (ctas <= tc::max_clusters_for(bn, swiglu != 0, s)) { splits = s; break; }
    }
  }
  const int per = (k_tiles + splits - 1) / splits;
  splits = (k_tiles + per - 1) / per;
  *bn_out = bn; *splits_out = splits; *live_y_out = live_y;
  return 0;
}

// x [T, K] bf16 (row stride ldx elements), w [G or 1][N or 2N][K] bf16 contiguous, out [*, N].
// `bn` and `splits` as cpi_gemm_tc_plan gives them (splits > 1 only with a power-of-two token tile up to 128).
extern "C" int cpi_gemm_tc(const void* x, long ldx, const void* w, void* out, int out_dtype, long ldo,
                           const int* out_rows, const float* row_scale, const int* group_offsets, int n_groups,
                           int T, int N, int K, int mode, int bn, int splits, int* error_flag,
                           cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  CPI_REQUIRE(T > 0 && N > 0 && K > 0, "gemm_tc: bad sizes T=%d N=%d K=%d", T, N, K);
  CPI_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_tc: K (%d) and the activation row stride (%ld) must be multiples of 8", K, ldx);
  CPI_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
              "gemm_tc: operands must be 16-byte aligned");
  CPI_REQUIRE(n_groups <= 256, "gemm_tc: %d groups (at most 256)", n_groups);
  CPI_REQUIRE(mode != tc::kAdd || out_dtype == kF32, "gemm_tc: ADD mode needs a float32 output");
  CPI_REQUIRE(mode != tc::kSwiglu || out_dtype == kBF16, "gemm_tc: SWIGLU mode writes bfloat16");
  const int acc = mode == tc::kSwiglu ? 2 : 1;
  const int rows_w = acc * N;
  const int groups = n_groups > 0 ? n_groups : 1;
  CUtensorMap mw, mx;
  if (tc::get_map(w, (uint64_t)K, (uint64_t)rows_w, (uint64_t)groups, (uint64_t)K * 2, (uint64_t)K * 2 * rows_w,
                  tc::BK, tc::BM, &mw)) return 1;
  if (tc::get_map(x, (uint64_t)K, (uint64_t)T, 0, (uint64_t)ldx * 2, 0, tc::BK, (uint32_t)(bn < 64 ? bn : 64), &mx)) return 1;   // bn < 64 is a power of two
  CPI_REQUIRE(bn >= 16 && bn <= 256 && bn % 16 == 0, "gemm_tc: token tile %d (multiples of 16 up to 256)", bn);
  int cap = 16;                                   // the compiled tile that holds bn rows
  while (cap < bn) cap *= 2;
  const int k_tiles = (K + tc::BK - 1) / tc::BK;
  const int per = (k_tiles + splits - 1) / splits;
  CPI_REQUIRE(splits >= 1 && (long)(splits - 1) * per < k_tiles, "gemm_tc: %d splits leave an empty split (k tiles %d)", splits, k_tiles);
  // token tiles: sum_g ceil(rows_g / bn) <= ceil(T / bn) + min(T, groups)
  dim3 grid((N + tc::BM - 1) / tc::BM, (T + bn - 1) / bn + (n_groups > 0 ? (T < n_groups ? T : n_groups) : 0), splits);
  CPI_REQUIRE(grid.y <= 65535, "gemm_tc: too many token tiles (%u)", grid.y);
  CPI_REQUIRE(splits == 1 || (splits <= 8 && bn == cap && cap <= 128),
              "gemm_tc: %d splits need a power-of-two token tile of at most 128 rows, got %d", splits, bn);
  // (measured on 16 experts: 5 % faster for the two-accumulator product at 2,048 tokens, slower for the
  // one-accumulator product, whose token rows are the larger operand)
  const int tiles_on_x = mode == tc::kSwiglu && n_groups > 0 && T > 2 * n_groups && splits == 1 && grid.x <= 65535;
  if (tiles_on_x) { const unsigned gx = grid.x; grid.x = grid.y; grid.y = gx; }
  tc::Params p{out, ldo, out_rows, row_scale, group_offsets, n_groups, T, bn, N, k_tiles, splits, per, tiles_on_x, error_flag, g_spin_limit, g_tx_extra};
  if (mode == tc::kStore && out_dtype == kBF16) return tc::launch_bn<tc::kStore, __nv_bfloat16>(cap, mw, mx, p, grid, stream);
  if (mode == tc::kStore && out_dtype == kF32) return tc::launch_bn<tc::kStore, float>(cap, mw, mx, p, grid, stream);
  if (mode == tc::kAdd) return tc::launch_bn<tc::kAdd, float>(cap, mw, mx, p, grid, stream);
  if (mode == tc::kSwiglu) return tc::launch_bn<tc::kSwiglu, __nv_bfloat16>(cap, mw, mx, p, grid, stream);
  set_error("gemm_tc: unsupported mode %d with output dtype %d", mode, out_dtype);
  return 1;
}
