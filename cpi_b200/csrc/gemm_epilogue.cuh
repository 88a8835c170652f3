// Epilogue of the tensor-core GEMMs for tiles with many token columns.
//
// The accumulator sits in tensor memory with the output FEATURE along the lanes (one thread each) and
// the TOKEN along the columns, while the output is [token][feature]: written straight from the
// registers, every store instruction of a warp covers only 32 features of one token (64 bytes of
// bfloat16), one instruction per token.  Measured on a 256 x 208 tile that cost 13 us (bf16 store) to
// 30 us (SwiGLU into rows 16 KB apart) against 2 us for reading tensor memory.  So the tile is turned
// in shared memory instead: each thread drops its feature's values at stage[token][feature] (a warp
// writes 32 neighbouring words: no bank conflicts), and after a barrier each warp copies whole token
// rows of 128 features with 16-byte (float32) or 8-byte (bfloat16) accesses per lane.  ADD of whole
// rows hands each turned row to the copy engine, which adds it into the output in the L2
// (cp.reduce.async.bulk, 512 bytes a row); a tile at the edge of N reads, adds and writes with several
// rows in flight.  Arithmetic and its order are those of the direct epilogue: out = old + acc * scale, or
// silu(g * scale) * (u * scale).
#pragma once
#include "common.cuh"

namespace cpi {
namespace epi {

enum Mode : int { kStore = 0, kAdd = 1, kSwiglu = 2 };

// silu(g) * u with the hardware's exponential and reciprocal (two special-function instructions and a few
// multiplies; relative error ~1e-7, far below the bfloat16 rounding of the result).  An exact division
// costs a dependent chain of ~30 instructions per element, which the four epilogue warps of a CTA cannot
// hide: on a 256-token tile it took longer than the tile's matrix product.  Every tensor-core epilogue
// uses this one function, so prefill and decode round alike.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <typename TO> struct Stage;
template <> struct Stage<float> {
  using T = float;
  static __device__ __forceinline__ float put(float v) { return v; }
};
template <> struct Stage<__nv_bfloat16> {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ __nv_bfloat16 put(float v) { return __float2bfloat16_rn(v); }
};

// Whether the staged epilogue may be used for this output: 128-feature rows of the tile start on
// 16-byte boundaries and the tile is wide enough for the detour to pay.
template <typename TO>
__device__ __forceinline__ bool staged_ok(const void* out, long ldo, int n_valid_t) {
  return n_valid_t >= 32 && (ldo % (16 / (int)sizeof(TO))) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
}

// ADD of whole float32 rows: the copy engine adds a turned row (128 features, 512 bytes of shared memory)
// into the output row in the L2, so no thread waits for the old values.  One writer per element and launch:
// the sum is old + acc as before.
__device__ __forceinline__ void bulk_add_f32(float* dst, const float* src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
               ::"l"(dst), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(src_smem))), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// Barriers of the turning: all threads of the CTA, or a named barrier over the calling threads only
// (a kernel whose other warps are busy with the next tile).
struct CtaSync { __device__ __forceinline__ void operator()() const { __syncthreads(); } };
template <int ID, int THREADS> struct NamedSync {
  __device__ __forceinline__ void operator()() const { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(THREADS) : "memory"); }
};

// ld16(col, dst): the caller's tensor-memory load of 16 columns starting at `col` of accumulator 0;
// ld16u the same for the second accumulator (SwiGLU).  `stage` holds STAGE_COLS x 128 elements of TO
// (STAGE_COLS a multiple of 16); a tile with more columns goes through in several passes.
// The 128 threads that own the accumulator's lanes call this; it contains barriers (`sync`).
template <int MODE, typename TO, int STAGE_COLS, typename Ld, typename LdU, typename Sync = CtaSync>
__device__ __forceinline__ void staged(void* stage_mem, Ld ld16, LdU ld16u, int warp, int lane, int n0, int N, int t0,
                                       int n_valid_t, int n_cols, TO* out, long ldo, const int* out_rows,
                                       const float* row_scale, Sync sync = Sync()) {
  static_assert(STAGE_COLS >= 16 && STAGE_COLS % 16 == 0, "the stage holds whole chunks of 16 columns");
  using S = typename Stage<TO>::T;
  S* stage = reinterpret_cast<S*>(stage_mem);
  const int row = warp * 32 + lane;                      // feature within the tile
  const float* scale = row_scale ? row_scale + t0 : nullptr;
  // Phase A.  Branch-free per chunk: the 16 values are computed side by side (one basic block, so their
  // special-function latencies overlap) and all are dropped into the stage; columns past the tile's
  // tokens hold zeros or finite junk and are never copied out.
  constexpr int PER = 4;                                 // features per lane: 32 lanes cover the 128 of a row
  constexpr int R = MODE == kAdd ? 16 : 8;              // rows in flight per warp (the read-modify-write waits on its loads)
  const int n = n0 + PER * lane;
  const bool whole = n + PER <= N;
  // all 128 features of the tile exist: rows leave through the copy engine's add (see bulk_add_f32)
  const bool bulk = MODE == kAdd && sizeof(TO) == 4 && n0 + 128 <= N &&
                    (reinterpret_cast<uintptr_t>(stage_mem) & 15) == 0;
#pragma unroll 1
  for (int p0 = 0; p0 < n_cols; p0 += STAGE_COLS) {      // one pass per STAGE_COLS columns
  const int p1 = min(p0 + STAGE_COLS, n_cols), v1 = min(p0 + STAGE_COLS, n_valid_t);
  if (p0 > 0) {
    if (bulk) bulk_wait_read();                          // the copy engine has read this thread's rows of the pass before
    sync();                                              // the previous pass has been copied out
  }
#pragma unroll 1
  for (int c = p0; c < p1; c += 16) {
    float v[16], u[16];
    ld16(c, v);
    if (MODE == kSwiglu) ld16u(c, u);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float s = scale ? scale[min(c + j, n_valid_t - 1)] : 1.0f;
      float x = v[j] * s;
      if (MODE == kSwiglu) x = silu_mul(x, u[j] * s);
      v[j] = x;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) stage[(c - p0 + j) * 128 + row] = Stage<TO>::put(v[j]);
  }
  if (bulk) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the stage is read through the async proxy
    sync();
    for (int col = p0 + row; col < v1; col += 128) {
      const int lr = t0 + col;
      bulk_add_f32(reinterpret_cast<float*>(out) + (size_t)(out_rows ? out_rows[lr] : lr) * ldo + n0,
                   reinterpret_cast<const float*>(stage) + (size_t)(col - p0) * 128, 512);
    }
    bulk_commit();
    continue;
  }
  sync();
  // Phase B.  A warp copies rows warp, warp + 4, ...; R rows per round, all their global loads first.
#pragma unroll 1
  for (int cb = p0 + warp; cb < v1; cb += 4 * R) {
    TO* dst[R];
    bool live[R];
#pragma unroll
    for (int q = 0; q < R; ++q) {
      const int col = cb + 4 * q;
      live[q] = col < v1;
      const int lr = t0 + (live[q] ? col : cb);
      dst[q] = out + (size_t)(out_rows ? out_rows[lr] : lr) * ldo + n;
    }
    if (sizeof(TO) == 4) {
      float4 old[R];
      if (MODE == kAdd) {
#pragma unroll
        for (int q = 0; q < R; ++q)
          if (live[q] && whole) old[q] = *reinterpret_cast<const float4*>(dst[q]);
      }
#pragma unroll
      for (int q = 0; q < R; ++q) {
        if (!live[q]) continue;
        const float4 sv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(stage) + ((cb + 4 * q) - p0) * 128 + PER * lane);
        if (whole) {
          float4 r = sv;
          if (MODE == kAdd) { r.x = old[q].x + r.x; r.y = old[q].y + r.y; r.z = old[q].z + r.z; r.w = old[q].w + r.w; }
          *reinterpret_cast<float4*>(dst[q]) = r;
        } else {
          const float e[4] = {sv.x, sv.y, sv.z, sv.w};
          float* d = reinterpret_cast<float*>(dst[q]);
          for (int i = 0; i < PER && n + i < N; ++i) d[i] = MODE == kAdd ? d[i] + e[i] : e[i];
        }
      }
    } else {
      uint2 sv[R];
#pragma unroll
      for (int q = 0; q < R; ++q)
        sv[q] = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(stage) + ((live[q] ? cb + 4 * q : cb) - p0) * 128 + PER * lane);
#pragma unroll
      for (int q = 0; q < R; ++q) {
        if (!live[q]) continue;
        if (whole) {
          *reinterpret_cast<uint2*>(dst[q]) = sv[q];
        } else {
          const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(&sv[q]);
          __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst[q]);
          for (int i = 0; i < PER && n + i < N; ++i) d[i] = src[i];
        }
      }
    }
  }
  }
  if (bulk) bulk_wait_read();                            // the stage may be written again; the sums land before the grid ends
}

}  // namespace epi
}  // namespace cpi
