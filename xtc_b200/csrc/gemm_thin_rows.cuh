// C[M,N] = A[M,K] x B[K,N] for a handful of rows (M <= 8): a matrix-vector product per row.
//
// Such a product reads B once and does two flops per element read: HBM bounds it, a tensor
// core tile of 128 rows would be 1/16 used at best, and the tile kernels' K loop per SM cannot
// pull B fast enough (1 x 4096 x 4096: 23 us on the tile kernels, 67 MB = 10 us of HBM time).
// Here every CTA streams a [K / 8, 64] block of B (128 columns wide when N >= 8192: fewer,
// longer runs per row of B) with plain 128-bit loads, four in flight per thread, and multiplies
// in fp32 on the CUDA cores (more exact than TF32, so every tolerance of the tensor-core path
// holds).  The eight K pieces of a column strip are the CTAs of one thread-block cluster: each
// reduces its 16 (or 8) row lanes in shared memory, then the CTA of rank 0 adds the eight
// partial rows in rank order through distributed shared memory and stores C.  No workspace, no
// atomics, the same bits on every run.
//
// Needs B row-major ([K, N], not the transposed form), N a multiple of 4, B and C 16-byte
// aligned with pitches that are multiples of 4; A may have either layout.
#pragma once
#include "common.cuh"

namespace xtc {

constexpr int THIN_THREADS = 256;
constexpr int THIN_COLS = 64;       // columns per CTA: 16 lanes of float4 and 16 row lanes, or
constexpr int THIN_COLS_WIDE = 128;  // 32 lanes of float4 and 8 row lanes (N >= 8192: longer runs per row)
constexpr int THIN_KSPLIT = 8;      // CTAs per cluster, one K piece each

struct ThinRowsParams {
  const float* A;
  const float* B;
  float* C;
  int M, N, K;
  long long lda, ldb, ldc;
  int a_t;  // A stored [K, M]
  int relu;
  float thr;
};

template <int MT, int COLS>
__global__ void __launch_bounds__(THIN_THREADS)
gemm_thin_rows_kernel(const ThinRowsParams p) {
  constexpr int ROW_LANES = THIN_THREADS * 4 / COLS;  // rows of B in flight per load round
  using namespace dev;
  extern __shared__ float thin_smem[];
  // [k in piece][MT] values of A, then [row lane][MT][COLS] partial sums, of which row
  // lane 0's block ends up holding the CTA's partial rows
  const uint32_t piece = cluster_ctarank();
  const int strip = blockIdx.x / THIN_KSPLIT;
  const int per_piece = (p.K + THIN_KSPLIT - 1) / THIN_KSPLIT;
  const int k0 = static_cast<int>(piece) * per_piece;
  const int k1 = k0 + per_piece < p.K ? k0 + per_piece : p.K;
  const int kn = k1 > k0 ? k1 - k0 : 0;
  float* a_s = thin_smem;
  float* red = thin_smem + ((static_cast<size_t>(per_piece) * MT + 3) & ~static_cast<size_t>(3));
  grid_dependency_sync();
  for (int i = threadIdx.x; i < kn * MT; i += THIN_THREADS) {
    const int k = i / MT, m = i - k * MT;
    float v = 0.f;
    if (m < p.M) v = p.a_t ? __ldg(p.A + static_cast<long long>(k0 + k) * p.lda + m)
                           : __ldg(p.A + static_cast<long long>(m) * p.lda + k0 + k);
    a_s[i] = v;
  }
  __syncthreads();

  constexpr int COL_GROUPS = COLS / 4;
  static_assert(COL_GROUPS * ROW_LANES == THIN_THREADS, "one float4 column group and row lane per thread");
  const int cl = threadIdx.x % COL_GROUPS;   // column group
  const int rl = threadIdx.x / COL_GROUPS;   // row lane
  const int col = strip * COLS + cl * 4;
  const bool col_ok = col < p.N;     // N is a multiple of 4: a group is inside or outside
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
  if (col_ok) {
    const float* bp = p.B + static_cast<long long>(k0) * p.ldb + col;
    int k = rl;
    // loads in flight per thread: with 4 or 8 rows of A a CTA holds 32 - 64 KB of shared memory,
    // fewer CTAs fit an SM, and each thread has to keep more of HBM's latency covered itself
    constexpr int DEPTH = MT >= 4 ? 8 : 4;
    for (; k + (DEPTH - 1) * ROW_LANES < kn; k += DEPTH * ROW_LANES) {
      float4 b[DEPTH];
#pragma unroll
      for (int u = 0; u < DEPTH; ++u)
        b[u] = __ldcs(reinterpret_cast<const float4*>(bp + static_cast<long long>(k + u * ROW_LANES) * p.ldb));
#pragma unroll
      for (int u = 0; u < DEPTH; ++u) {
        const float* ar = a_s + (k + u * ROW_LANES) * MT;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float a = ar[m];
          acc[m][0] = fmaf(a, b[u].x, acc[m][0]);
          acc[m][1] = fmaf(a, b[u].y, acc[m][1]);
          acc[m][2] = fmaf(a, b[u].z, acc[m][2]);
          acc[m][3] = fmaf(a, b[u].w, acc[m][3]);
        }
      }
    }
    for (; k < kn; k += ROW_LANES) {
      const float4 b = __ldcs(reinterpret_cast<const float4*>(bp + static_cast<long long>(k) * p.ldb));
      const float* ar = a_s + k * MT;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float a = ar[m];
        acc[m][0] = fmaf(a, b.x, acc[m][0]);
        acc[m][1] = fmaf(a, b.y, acc[m][1]);
        acc[m][2] = fmaf(a, b.z, acc[m][2]);
        acc[m][3] = fmaf(a, b.w, acc[m][3]);
      }
    }
  }
  // the 16 row lanes of this CTA, summed in lane order by the threads of row lane 0
#pragma unroll
  for (int m = 0; m < MT; ++m)
    *reinterpret_cast<float4*>(red + (static_cast<size_t>(rl) * MT + m) * COLS + cl * 4) =
        make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  __syncthreads();
  if (rl == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float4 s = *reinterpret_cast<const float4*>(red + static_cast<size_t>(m) * COLS + cl * 4);
      for (int r = 1; r < ROW_LANES; ++r) {
        const float4 v = *reinterpret_cast<const float4*>(red + (static_cast<size_t>(r) * MT + m) * COLS + cl * 4);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      *reinterpret_cast<float4*>(red + static_cast<size_t>(m) * COLS + cl * 4) = s;
    }
  }
  cluster_sync_all();  // every piece's partial rows are in place
  if (piece == 0 && rl == 0 && col_ok) {
    const uint32_t mine = smem_u32(red + cl * 4);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m >= p.M) break;
      float4 s = *reinterpret_cast<const float4*>(red + static_cast<size_t>(m) * COLS + cl * 4);
      for (uint32_t r = 1; r < THIN_KSPLIT; ++r) {
        const float4 v = ld_shared_cluster_f4(map_to_cta(mine + static_cast<uint32_t>(m) * COLS * 4, r));
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      if (p.relu) {
        s.x = fmaxf(s.x, p.thr); s.y = fmaxf(s.y, p.thr);
        s.z = fmaxf(s.z, p.thr); s.w = fmaxf(s.w, p.thr);
      }
      *reinterpret_cast<float4*>(p.C + static_cast<long long>(m) * p.ldc + col) = s;
    }
  }
  cluster_sync_all();  // no CTA leaves while rank 0 may still read its shared memory
}

// Shared memory one CTA needs for M rows (rounded up to 1, 2, 4 or 8) and a K of `K`.
inline size_t thin_rows_smem(int mt, long long K) {
  const size_t per_piece = static_cast<size_t>((K + THIN_KSPLIT - 1) / THIN_KSPLIT);
  return (((per_piece * mt + 3) & ~static_cast<size_t>(3)) +
          static_cast<size_t>(THIN_THREADS) * 4 * mt) * sizeof(float);  // row lanes x columns = 4 x threads
}

}  // namespace xtc
