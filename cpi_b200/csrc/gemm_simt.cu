// General matrix product on the FP32 pipe (FFMA): out[m, n] = sum_k A[row(m), k] * W[g(m)][n, k].
//
// This is the true 32-bit contraction of the library: float accumulation in a fixed k order
// (no tensor cores, no tf32), for any mix of float32 / bfloat16 activations and weights (bfloat16
// widens exactly, as src/engine/llama4_cpu_engine.cpp:24-29 does).  The bfloat16 path uses it for
// shapes that the tensor-core kernels refuse.  The reference's counterparts are its GEMV kernels
// (src/kernels/kernels_ops_matvec.cu:343-418) and one cublasGemmEx call
// (src/engine/llama4_cuda_engine_setup.cu:579-605), all batch 1.
//
// Modes:  STORE   out = acc * scale(m)
//         ADD     out += acc * scale(m)                      (out is the float32 residual stream)
//         SWIGLU  out = silu(g) * u,  g = scale(m) * sum_k A W[n, k],  u = scale(m) * sum_k A W[N + n, k]
// Optional row gather (a_rows), output row scatter (out_rows), per-row scale, and groups: logical
// rows [offsets[g], offsets[g+1]) use the weight matrix W + g * w_group_stride (routed experts).
#include "common.cuh"

namespace cpi {

enum GemmMode : int { kStore = 0, kAdd = 1, kSwiglu = 2 };

struct GemmParams {
  const void* a; long lda; const int* a_rows;
  const void* w; long ldw; long w_group_stride;
  void* out; long ldo; const int* out_rows;
  const float* row_scale;
  const int* group_offsets; int n_groups;
  int M, N, K;
};

constexpr int BN = 64, BK = 16, NT = 256;

template <typename TA, typename TW, typename TO, int MODE, int TM>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(GemmParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int BM = 16 * TM;
  constexpr bool GLU = MODE == kSwiglu;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[GLU ? 2 : 1][BK][BN + 4];

  int m_begin = 0, m_end = p.M;
  const TW* w = reinterpret_cast<const TW*>(p.w);
  int tile_m = blockIdx.y;
  if (p.group_offsets) {
    // map blockIdx.y to (group, tile in group): groups are visited in order
    int g = 0, found = 0;
    for (; g < p.n_groups; ++g) {
      const int b = p.group_offsets[g], e = p.group_offsets[g + 1];
      const int tiles = (e - b + BM - 1) / BM;
      if (tile_m < tiles) { m_begin = b; m_end = e; found = 1; break; }
      tile_m -= tiles;
    }
    if (!found) return;
    w += (size_t)g * p.w_group_stride;
  }
  const int m0 = m_begin + tile_m * BM;
  if (m0 >= m_end) return;
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  float acc[TM][4], acc2[GLU ? TM : 1][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; if (GLU) acc2[i][j] = 0.f; }

  const TA* a = reinterpret_cast<const TA*>(p.a);
  // loader mapping: A tile BM x BK, 4 consecutive k per thread
  const int la_row = tid >> 2, la_k = (tid & 3) * 4;        // valid for tid < BM*4
  const bool la_active = la_row < BM && (m0 + la_row) < m_end;
  const TA* a_ptr = nullptr;
  if (la_active) {
    const int lr = m0 + la_row;
    a_ptr = a + (size_t)(p.a_rows ? p.a_rows[lr] : lr) * p.lda;
  }
  const int lw_row = tid >> 2, lw_k = (tid & 3) * 4;          // W tile BN x BK: 64 rows x 4 threads
  const bool lw_active = (n0 + lw_row) < p.N;
  const TW* w_ptr = w + (size_t)(n0 + lw_row) * p.ldw;
  const TW* w2_ptr = w + (size_t)(p.N + n0 + lw_row) * p.ldw;

  for (int k0 = 0; k0 < p.K; k0 += BK) {
    if (la_row < BM) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = k0 + la_k + j;
        As[la_k + j][la_row] = (la_active && k < p.K) ? to_f32(a_ptr[k]) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lw_k + j;
      const bool ok = lw_active && k < p.K;
      Ws[0][lw_k + j][lw_row] = ok ? to_f32(w_ptr[k]) : 0.f;
      if (GLU) Ws[1][lw_k + j][lw_row] = ok ? to_f32(w2_ptr[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[TM], wv[4], wv2[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) { wv[j] = Ws[0][k][tx * 4 + j]; if (GLU) wv2[j] = Ws[1][k][tx * 4 + j]; }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if (GLU) acc2[i][j] = fmaf(av[i], wv2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }

  TO* out = reinterpret_cast<TO*>(p.out);
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int lr = m0 + ty * TM + i;
    if (lr >= m_end) continue;
    const float s = p.row_scale ? p.row_scale[lr] : 1.0f;
    TO* o = out + (size_t)(p.out_rows ? p.out_rows[lr] : lr) * p.ldo;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j] * s;
      if (MODE == kSwiglu) {
        const float u = acc2[i][j] * s;
        v = v / (1.0f + expf(-v)) * u;
        o[n] = from_f32<TO>(v);
      } else if (MODE == kAdd) {
        o[n] = from_f32<TO>(to_f32(o[n]) + v);
      } else {
        o[n] = from_f32<TO>(v);
      }
    }
  }
}

template <typename TA, typename TW, typename TO, int MODE>
int launch_simt(const GemmParams& p, int m_tiles_hint, cudaStream_t stream) {
  // rows per tile: 16 when few rows are expected per group, else 64
  const bool small = m_tiles_hint <= 16;
  const int BM = small ? 16 : 64;
  int m_tiles = (p.M + BM - 1) / BM;
  if (p.group_offsets) m_tiles += p.n_groups;
  dim3 grid((p.N + BN - 1) / BN, m_tiles);
  if (grid.y > 65535) { set_error("gemm: too many row tiles (%u)", grid.y); return 1; }
  if (small) cpi::launch_pdl(gemm_simt_kernel<TA, TW, TO, MODE, 1>, grid, NT, 0, stream, p);
  else       cpi::launch_pdl(gemm_simt_kernel<TA, TW, TO, MODE, 4>, grid, NT, 0, stream, p);
  return check_launch("gemm_simt");
}

template <typename TA, typename TW, typename TO>
int launch_mode(const GemmParams& p, int mode, int hint, cudaStream_t s) {
  switch (mode) {
    case kStore:  return launch_simt<TA, TW, TO, kStore>(p, hint, s);
    case kAdd:    return launch_simt<TA, TW, TO, kAdd>(p, hint, s);
    case kSwiglu: return launch_simt<TA, TW, TO, kSwiglu>(p, hint, s);
  }
  set_error("gemm: unknown mode %d", mode);
  return 1;
}

}  // namespace cpi

using namespace cpi;

// a [*, K] (lda), w [N or 2N (SWIGLU), K] (ldw) per group, out [*, N] (ldo).
// M = number of logical rows (over all groups); rows_per_group_hint sizes the row tile.
extern "C" int cpi_gemm_simt(const void* a, int a_dtype, long lda, const int* a_rows,
                             const void* w, int w_dtype, long ldw, long w_group_stride,
                             void* out, int out_dtype, long ldo, const int* out_rows,
                             const float* row_scale, const int* group_offsets, int n_groups,
                             int M, int N, int K, int mode, int rows_per_group_hint, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  CPI_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  CPI_REQUIRE(mode != kAdd || out_dtype == kF32, "gemm: ADD mode needs a float32 output");
  GemmParams p{a, lda, a_rows, w, ldw, w_group_stride, out, ldo, out_rows, row_scale,
               group_offsets, n_groups, M, N, K};
  CPI_DISPATCH_DTYPE(a_dtype, TA, CPI_DISPATCH_DTYPE(w_dtype, TW, CPI_DISPATCH_DTYPE(out_dtype, TO,
      return (launch_mode<TA, TW, TO>(p, mode, rows_per_group_hint, stream)))));
  return 0;
}
