// Prefill attention in bfloat16 on tcgen05: two tiles of 128 queries of one head against the paged cache.
//
// A CTA owns up to 256 consecutive tokens of one sequence and one query head: query tile A (the first 128
// rows) and query tile B (the rest).  Warp 8 streams key/value tiles (128 positions = two cache pages, through
// TMA with the 128-byte swizzle) into a ring of five shared-memory slots, K(i), V(i), K(i+1), ...: both query
// tiles use every key and value tile, so each is fetched once for 256 queries.  One thread of warp 9 issues
// the MMAs; warps 0-3 are the softmax of tile A, warps 4-7 of tile B: thread r of a group owns query row r
// and all 128 key columns of a tile, so row maxima and sums need no shuffles.  Per key tile and query tile:
//     S = Q K^T            tcgen05.mma, both operands K-major from shared memory, S in tensor memory
//     P = 2^(S*c - m)      read S with tcgen05.ld, mask by position, write P as bf16 over the first 64 columns
//                          of the S it came from
//     O += P V             tcgen05.mma with P as the A operand from tensor memory, accumulating in tensor
//                          memory; V consumed MN-major straight from the page layout [position][dim]
// Tensor memory holds S and O of both query tiles (4 x 128 columns).  The products of the two tiles alternate
// in the issue order (P_A V, Q_A K'^T, P_B V, Q_B K'^T), so the tensor pipe works for one tile while the
// other's softmax runs; the exponentials of a tile (16,384 on 16 per cycle) take as long as its two products.
// m is a reference maximum that is raised, and O rescaled in tensor memory, only when the row maximum
// has outgrown it by 2^8; the division by the row sum comes once, at the end.
// Masks: key position <= query position, and >= the window's low end (chunk or sliding window).  The
// last tile's value rows beyond the newest position are zeroed in shared memory, so stale page contents
// cannot reach the product (0 * NaN).  Formulas: src/engine/llama4_cpu_engine.cpp:195-250; the
// reference's own prefill is a loop of single-token forwards (src/engine/llama4_cuda_engine.cu:571-580).
//
// Every mbarrier wait is bounded; when one runs out the CTA sets *error_flag and leaves.
#include "common.cuh"
#include <cuda.h>

namespace cpi {
namespace tc {
// from gemm_tc.cu
int get_map_2d_bf16(const void* ptr, uint64_t inner, uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner,
                    uint32_t box_rows, CUtensorMap* out);
}
namespace pre {

constexpr int BQ = 128, BKV = 128, PAGE = 64;
constexpr uint32_t kSpinLimit = 1u << 24;

struct Params {
  __nv_bfloat16* out;                 // [T, NH * D]
  const int* page_table; int max_blocks;
  const int* token_pos; const int* token_seq; const int* seq_slot;
  const int* tile_tok0; const int* tile_rows;     // per query tile: first packed token, valid rows
  int n_heads, n_kv_heads;
  int window_kind, window_size;
  float scale_log2;
  int* error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// the same with the A operand (M x 16 bfloat16, two per 32-bit column) in tensor memory
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// One lane of a converged warp.  The warp that issues the MMAs runs its loop with all 32 lanes (so that the
// compiler sees uniform values and keeps descriptors and loop counters on the uniform datapath) and only
// the tcgen05 instructions themselves sit under this predicate.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// accumulate known at compile time: no run-time predicate set-up per instruction
template <bool ACC>
__device__ __forceinline__ void umma_bf16_c(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc) {
  if (ACC)
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc) : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc) : "memory");
}
template <bool ACC>
__device__ __forceinline__ void umma_bf16_a_tmem_c(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc) {
  if (ACC)
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc) : "memory");
  else
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc) : "memory");
}
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// the same load without the wait: the caller overlaps it with arithmetic on the chunk before
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// shared-memory matrix descriptor, 128-byte swizzle; lbo/sbo in bytes
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ int window_low(int kind, int size, int pos) {
  if (kind == 1) return (pos / size) * size;
  if (kind == 2) return max(0, pos - size + 1);
  return 0;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
        "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
        "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 16 packed columns (32 bfloat16 of this thread's row) into tensor memory; the caller waits once per pass
__device__ __forceinline__ void tmem_st16_nowait(uint32_t taddr, const uint32_t* w) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]),
        "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Exponentials are taken against a reference maximum that is only raised when the true row maximum has
// outgrown it by more than this many powers of two; the accumulated output then needs rescaling only
// then (rarely after the first tiles), and intermediate values stay below 2^kRescaleSlack.
constexpr float kRescaleSlack = 8.0f;
constexpr int kRingSlots = 5;           // key and value tiles in shared memory at a time
constexpr int kTileRows = 2 * BQ;       // query rows a CTA takes: two tiles of 128

template <int D>
__global__ void __launch_bounds__(320) attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                const __grid_constant__ CUtensorMap map_k,
                                                                const __grid_constant__ CUtensorMap map_v, Params p) {
  constexpr int HALVES = D / 64;                       // 64-element (128-byte) column blocks of a row
  constexpr uint32_t HALF_BYTES = 128 * 128;           // 128 rows x 128 bytes
  constexpr uint32_t Q_BYTES = HALVES * HALF_BYTES;    // one query tile of 128 rows
  constexpr uint32_t KV_BYTES = HALVES * HALF_BYTES;   // one of K or V, 128 positions
  constexpr uint32_t TMEM_COLS = 512;                  // S of tile A, S of tile B (128 columns each), O of A, O of B
  constexpr int NSLOT = kRingSlots;                    // ring of key and value tiles: K(i), V(i), K(i+1), ...
  // (aligned by declaration: with head size 128 the tiles fill what an SM has, there is no room for slack)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t q_full, kv_full[NSLOT], kv_empty[NSLOT], s_full[2], p_full[2], o_done[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* q_s = smem_raw;                             // [2 query tiles]
  uint8_t* ring = q_s + 2 * Q_BYTES;                   // [NSLOT]

  pdl_launch_dependents();
  pdl_wait();
  const int tile = blockIdx.y, head = blockIdx.x;       // heads are the fast axis: all heads of the longest tile start first
  const int kvh = head / (p.n_heads / p.n_kv_heads);
  const int tok0 = p.tile_tok0[tile], rows = p.tile_rows[tile];
  const int slot = p.seq_slot[p.token_seq[tok0]];
  // the tile's rows are consecutive positions of one sequence; rows 0-127 are query tile A, the rest tile B
  const int pos_first = p.token_pos[tok0], pos_last = pos_first + rows - 1;
  const int rows_x[2] = {min(rows, BQ), max(rows - BQ, 0)};
  const bool has_b = rows_x[1] > 0;
  const int p0_x[2] = {pos_first, pos_first + BQ};                         // first position of A, of B
  const int p1_x[2] = {pos_first + rows_x[0] - 1, pos_last};               // last position of A, of B
  // key tiles (of 128 positions) that each query tile meets; the window's low end never decreases with the position
  const int kb_x[2] = {window_low(p.window_kind, p.window_size, p0_x[0]) / BKV,
                       has_b ? window_low(p.window_kind, p.window_size, p0_x[1]) / BKV : 0};
  const int ke_x[2] = {p1_x[0] / BKV + 1, has_b ? p1_x[1] / BKV + 1 : 0};
  const int kt0 = kb_x[0], kt1 = has_b ? ke_x[1] : ke_x[0];               // the union: every tile in it is met by A or B

  if (tid == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < NSLOT; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4); mbar_init(&o_done[s], 1);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 256;        // + 128 for tile B, both
  volatile int* abort_flag = &abort_s;
  bool ok = true;

  if (warp == 8) {
    if (lane == 0) {
      // ---- TMA producer: Q of both tiles, then K(kt0), V(kt0), K(kt0 + 1), ... through the ring ----
      mbar_expect_tx(&q_full, Q_BYTES * (has_b ? 2 : 1));
      for (int x = 0; x < (has_b ? 2 : 1); ++x)
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(q_s + x * Q_BYTES + h * HALF_BYTES, &map_q, &q_full, head * D + h * 64, tok0 + x * BQ);
      const int* table = p.page_table + (size_t)slot * p.max_blocks;
      const int last_block = pos_last / PAGE;
      int n = 0;                                         // item of the ring: 2 (kt - kt0) for keys, + 1 for values
      for (int kt = kt0; kt < kt1 && ok; ++kt) {
        const int blk0 = kt * (BKV / PAGE);
        const int n_pages = min(BKV / PAGE, last_block - blk0 + 1);
        const uint32_t bytes = (uint32_t)n_pages * HALVES * (PAGE * 128);
        for (int which = 0; which < 2; ++which, ++n) {
          const int s = n % NSLOT;
          if (n >= NSLOT && !mbar_wait(&kv_empty[s], ((n / NSLOT) - 1) & 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&kv_full[s], bytes);
          for (int pg = 0; pg < n_pages; ++pg) {
            const int row = (table[blk0 + pg] * p.n_kv_heads + kvh) * PAGE;
            for (int h = 0; h < HALVES; ++h)
              tma_load_2d(ring + s * KV_BYTES + h * HALF_BYTES + pg * (PAGE * 128), which ? &map_v : &map_k,
                          &kv_full[s], h * 64, row);
          }
        }
      }
    }
  } else if (warp == 9) {
    // ---- MMA issuer.  Two query tiles share every key and value tile.  Per key tile kt:
    //          O_A += P_A V(kt);  S_A = Q_A K(kt+1)^T;   O_B += P_B V(kt);  S_B = Q_B K(kt+1)^T
    //      so that while the softmax threads of one query tile work on its S, the tensor pipe runs the other
    //      tile's products.  P is written over the S it came from (as bf16, the first 64 columns) and is the
    //      A operand of P V from tensor memory; the next Q K^T of the same query tile is issued after that
    //      P V and the pipe runs in issue order, so it cannot overwrite a P that is still being read.
    //      The whole warp runs the loop (uniform values stay on the uniform datapath); only the tcgen05
    //      instructions sit under the elected lane. ----
    constexpr uint32_t idesc_s = instr_desc(BQ, BKV, 0);
    constexpr uint32_t idesc_o = instr_desc(BQ, D, 1);
    constexpr uint64_t kSlotUnits = KV_BYTES >> 4;      // a ring slot further, in the descriptor's 16-byte units
    const uint64_t dq[2] = {smem_desc(smem_u32(q_s), 16, 1024), smem_desc(smem_u32(q_s + Q_BYTES), 16, 1024)};
    const uint64_t dk0 = smem_desc(smem_u32(ring), 16, 1024), dv0 = smem_desc(smem_u32(ring), HALF_BYTES, 1024);
    // Everything the loop needs is a counter that is advanced by additions (this warp shares its scheduler with
    // two softmax warps: every instruction between two MMAs is time the tensor pipe stands still).  Ring slot
    // and phase of the next key tile and of the next value tile to be used, per query tile:
    int ks[2], kph[2], vs[2], vph[2], pph[2] = {0, 0}, first_pv[2] = {1, 1};
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const int nk = 2 * (kb_x[x] - kt0), nv = nk + 1;
      ks[x] = nk % NSLOT; kph[x] = (nk / NSLOT) & 1;
      vs[x] = nv % NSLOT; vph[x] = (nv / NSLOT) & 1;
    }
    // S_x = Q_x K^T on the key tile in ring slot ks[x]; `release`: no later product reads that key tile
    auto issue_qk = [&](int x, bool release) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(&kv_full[ks[x]], kph[x], abort_flag))) return false;
      fence_after_sync();
      if (elect_one()) {
        const uint64_t dk = dk0 + (uint64_t)ks[x] * kSlotUnits;
        umma_bf16_c<false>(tmem_s + x * 128, dq[x], dk, idesc_s);
#pragma unroll
        for (int k = 1; k < D / 16; ++k) {
          const uint64_t off = (uint64_t)(((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4);
          umma_bf16_c<true>(tmem_s + x * 128, dq[x] + off, dk + off, idesc_s);
        }
        umma_commit(&s_full[x]);
        if (release) umma_commit(&kv_empty[ks[x]]);
      }
      __syncwarp();
      ks[x] += 2;                                        // the next key tile is two ring items further
      if (ks[x] >= NSLOT) { ks[x] -= NSLOT; kph[x] ^= 1; }
      return true;
    };
    // O_x += P_x V on the value tile in ring slot vs[x]
    auto issue_pv = [&](int x, bool release) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(&p_full[x], pph[x], abort_flag) &&
                                       mbar_wait(&kv_full[vs[x]], vph[x], abort_flag))) return false;
      fence_after_sync();
      if (elect_one()) {
        const uint64_t dv = dv0 + (uint64_t)vs[x] * kSlotUnits;
        const uint32_t pa = tmem_s + x * 128, od = tmem_o + x * 128;
        if (first_pv[x]) umma_bf16_a_tmem_c<false>(od, pa, dv, idesc_o);
        else umma_bf16_a_tmem_c<true>(od, pa, dv, idesc_o);
#pragma unroll
        for (int j = 1; j < BKV / 16; ++j)
          umma_bf16_a_tmem_c<true>(od, pa + j * 8, dv + (uint64_t)(j * (2048 >> 4)), idesc_o);
        if (release) umma_commit(&kv_empty[vs[x]]);
      }
      __syncwarp();
      first_pv[x] = 0;
      pph[x] ^= 1;
      vs[x] += 2;
      if (vs[x] >= NSLOT) { vs[x] -= NSLOT; vph[x] ^= 1; }
      return true;
    };
    ok = __all_sync(0xffffffffu, mbar_wait(&q_full, 0, abort_flag));
    const int kb_b = has_b ? kb_x[1] : 0x7fffffff, ke_a = ke_x[0];
    ok = ok && issue_qk(0, kb_b != kt0);
    if (ok && kb_b == kt0) ok = issue_qk(1, true);
    for (int kt = kt0; kt < kt1 && ok; ++kt) {
      // which query tiles meet key tile kt, and kt + 1 (B's range ends with the union's, A's begins with it)
      const bool a_now = kt < ke_a, b_now = kt >= kb_b;
      const bool a_next = kt + 1 < ke_a, b_next = kt + 1 >= kb_b && kt + 1 < kt1;
      if (a_now) {
        ok = issue_pv(0, !b_now);
        if (ok && a_next) ok = issue_qk(0, !b_next);
      }
      if (ok && b_now) ok = issue_pv(1, true);
      if (ok && b_next) ok = issue_qk(1, true);
    }
    // every product has been issued: one arrival says that O of both query tiles is complete
    if (ok && elect_one()) { umma_commit(&o_done[0]); umma_commit(&o_done[1]); }
    __syncwarp();
  } else {
    // ---- softmax: warps 0-3 own query tile A, warps 4-7 tile B; thread r of a group owns query row r and all
    //      128 key columns of a tile (a warp may touch the 32 lanes of tensor memory given by its number modulo
    //      4).  Row maxima and sums need no shuffles, and the maximum is exact before any exponential is taken.
    //      O stays in tensor memory and is rescaled only when a row maximum has outgrown its reference. ----
    const int x = warp >> 2, row = tid & 127;
    const bool live = row < rows_x[x];
    const int qp = live ? p0_x[x] + row : -1;
    const int lo = live ? window_low(p.window_kind, p.window_size, qp) : 0;
    const int lo_last = window_low(p.window_kind, p.window_size, p1_x[x]);
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_row = tmem_s + x * 128 + lane_addr, o_row = tmem_o + x * 128 + lane_addr;
    float m_ref = -1e30f, l_run = 0.f;                  // reference maximum of the exponentials; the row's sum
    const float sc = p.scale_log2;                      // > 0: the maximum may be taken before scaling
    // the union's last key tile holds positions beyond the newest one: their value rows are zeroed by the group
    // whose P V on that tile is issued first (A if it meets the tile, otherwise B)
    const bool zero_duty = x == 0 ? (kt1 - 1 >= kb_x[0] && kt1 - 1 < ke_x[0]) : !(kt1 - 1 >= kb_x[0] && kt1 - 1 < ke_x[0]);
    int j = 0;
    bool okl = rows_x[x] > 0;
    for (int kt = kb_x[x]; kt < ke_x[x] && okl; ++kt, ++j) {
      const int key0 = kt * BKV;
      // (tensor-memory loads and votes are warp-wide: a warp gives up as a whole)
      okl = __all_sync(0xffffffffu, mbar_wait(&s_full[x], j & 1, abort_flag));
      if (okl && kt == kt1 - 1 && zero_duty) {
        const int n = 2 * (kt - kt0) + 1, sl = n % NSLOT;
        okl = __all_sync(0xffffffffu, mbar_wait(&kv_full[sl], (n / NSLOT) & 1, abort_flag));
        if (okl && key0 + row > pos_last) {
          uint8_t* vs = ring + sl * KV_BYTES;
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            uint4* r4 = reinterpret_cast<uint4*>(vs + h * HALF_BYTES + row * 128);
#pragma unroll
            for (int q = 0; q < 8; ++q) r4[q] = make_uint4(0, 0, 0, 0);
          }
        }
        fence_async_proxy();                             // the MMA reads V through the async proxy
      }
      if (!okl) break;
      fence_after_sync();
      // a tile that lies wholly inside every row's window needs no position tests
      const bool no_mask = key0 + BKV - 1 <= p0_x[x] && key0 >= lo_last;
      // One pass over the row's 128 columns of S, 32 at a time with the next chunk's load in flight: the
      // maximum, P = 2^(s c - ref) as packed bf16, and the sum.  P is kept in registers until the pass is
      // known to stand, because it goes over the S it came from.
      uint32_t w[BKV / 32][16];
      float mx, ls;
      auto pass = [&](const float ref) {
        const float nref = -ref;
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, ls4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t raw[2][32];
        tmem_ld32_issue(s_row, raw[0]);
        tmem_ld32_issue(s_row + 32, raw[1]);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < BKV / 32; ++cc) {
          float v[32];
          if (no_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float sv = __uint_as_float(raw[cc & 1][e]);
              mx4[e & 3] = fmaxf(mx4[e & 3], sv);
              v[e] = exp2_fast(fmaf(sv, sc, nref));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int kp = key0 + cc * 32 + e;
              const bool in = kp <= qp && kp >= lo;
              const float sv = __uint_as_float(raw[cc & 1][e]);
              if (in) mx4[e & 3] = fmaxf(mx4[e & 3], sv);
              v[e] = in ? exp2_fast(fmaf(sv, sc, nref)) : 0.f;
            }
          }
          if (cc + 2 < BKV / 32) tmem_ld32_issue(s_row + (cc + 2) * 32, raw[cc & 1]);     // this buffer is consumed
#pragma unroll
          for (int e = 0; e < 32; ++e) ls4[e & 3] += v[e];
#pragma unroll
          for (int g = 0; g < 16; ++g) w[cc][g] = pack_bf16(v[2 * g], v[2 * g + 1]);
          if (cc == 1) tmem_wait_ld();
        }
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;
        ls = (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      };
      // Optimistic: against the reference maximum the row already has.  Only if some row of the warp has
      // outgrown its reference by more than the slack (always on its first tile) is the reference raised, O
      // rescaled in tensor memory, and the pass repeated: S is still whole, nothing has been stored yet.
      pass(m_ref);
      const bool grow = mx > m_ref + (m_ref < -1e29f ? 0.f : kRescaleSlack);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : m_ref;
        const float f = exp2f(m_ref - m_new);
        if (j > 0) {
          // Every P V issued so far for this query tile has landed: the Q K^T whose S was waited for above was
          // issued after the last of them, and its arrival covers everything issued before it.
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            float v[32];
            tmem_ld32(o_row + c, v);
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] *= f;
            tmem_st32(o_row + c, v);
          }
        }
        l_run *= f;
        m_ref = m_new;
        pass(m_ref);
      }
#pragma unroll
      for (int cc = 0; cc < BKV / 32; ++cc) tmem_st16_nowait(s_row + cc * 16, w[cc]);
      l_run += ls;
      tmem_wait_st();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);            // one arrival per warp
    }
    // the output: O / l once the last P V is done
    ok = okl && !abort_s && j > 0;
    ok = __all_sync(0xffffffffu, ok && mbar_wait(&o_done[x], 0, abort_flag));
    fence_after_sync();
    if (ok) {
      const float inv = 1.0f / fmaxf(l_run, 1e-20f);
      __nv_bfloat16* dst = p.out + ((size_t)(tok0 + x * BQ + row) * p.n_heads + head) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        float v[32];
        tmem_ld32(o_row + c, v);
        if (live) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w = make_uint4(pack_bf16(v[e] * inv, v[e + 1] * inv), pack_bf16(v[e + 2] * inv, v[e + 3] * inv),
                                 pack_bf16(v[e + 4] * inv, v[e + 5] * inv), pack_bf16(v[e + 6] * inv, v[e + 7] * inv));
            *reinterpret_cast<uint4*>(dst + c + e) = w;
          }
        }
      }
    }
    fence_before_sync();
  }
  if (abort_s) {
    if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 2);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(TMEM_COLS));
}

}  // namespace pre
}  // namespace cpi

using namespace cpi;

extern "C" int cpi_attention_prefill_tile_rows() { return pre::kTileRows; }

extern "C" int cpi_attention_prefill_supported(int n_heads, int n_kv_heads, int head_dim, int page_size) {
  if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
  return (head_dim == 64 || head_dim == 128) && page_size == pre::PAGE;
}

// q, out [T, NH*D] bfloat16; k_cache, v_cache [n_pages, NKV, 64, D] bfloat16 of one layer.
// tile_tok0 / tile_rows (device, int32 [n_tiles]): first packed token and valid rows (1..256, see
// cpi_attention_prefill_tile_rows) of each CTA's queries; they belong to one sequence and have consecutive
// positions.
extern "C" int cpi_attention_prefill(const void* q, void* out, const void* k_cache, const void* v_cache, long n_pages,
                                     const int* page_table, int max_blocks, int page_size, const int* token_seq,
                                     const int* token_pos, const int* seq_slot, const int* tile_tok0,
                                     const int* tile_rows, int n_tiles, int n_tokens, int n_heads, int n_kv_heads,
                                     int head_dim, int window_kind, int window_size, float scale, int* error_flag,
                                     cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  CPI_REQUIRE(cpi_attention_prefill_supported(n_heads, n_kv_heads, head_dim, page_size),
              "attention_prefill: unsupported shape (heads %d/%d, head size %d, page %d)", n_heads, n_kv_heads, head_dim, page_size);
  CPI_REQUIRE(window_kind == 0 || window_size > 0, "attention_prefill: window kind %d needs a size > 0", window_kind);
  CPI_REQUIRE(n_tiles <= 65535, "attention_prefill: too many query tiles in one launch (%d)", n_tiles);
  CUtensorMap mq, mk, mv;
  const uint64_t q_width = (uint64_t)n_heads * head_dim;
  if (tc::get_map_2d_bf16(q, q_width, (uint64_t)n_tokens, q_width * 2, 64, pre::BQ, &mq)) return 1;
  const uint64_t kv_rows = (uint64_t)n_pages * n_kv_heads * pre::PAGE;
  if (tc::get_map_2d_bf16(k_cache, (uint64_t)head_dim, kv_rows, (uint64_t)head_dim * 2, 64, pre::PAGE, &mk)) return 1;
  if (tc::get_map_2d_bf16(v_cache, (uint64_t)head_dim, kv_rows, (uint64_t)head_dim * 2, 64, pre::PAGE, &mv)) return 1;
  pre::Params p{(__nv_bfloat16*)out, page_table, max_blocks, token_pos, token_seq, seq_slot, tile_tok0, tile_rows,
                n_heads, n_kv_heads, window_kind, window_size, scale * 1.4426950408889634f, error_flag};
  dim3 grid(n_heads, n_tiles);
  const int halves = head_dim / 64;
  const int smem = halves * 128 * 128 * (2 + pre::kRingSlots);     // Q of both tiles, the ring of K and V tiles
  if (head_dim == 128) {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(pre::attention_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); set = true; }
    cpi::launch_pdl(pre::attention_prefill_kernel<128>, grid, 320, smem, stream, mq, mk, mv, p);
  } else {
    static bool set = false;
    if (!set) { cudaFuncSetAttribute(pre::attention_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); set = true; }
    cpi::launch_pdl(pre::attention_prefill_kernel<64>, grid, 320, smem, stream, mq, mk, mv, p);
  }
  return check_launch("attention_prefill");
}
