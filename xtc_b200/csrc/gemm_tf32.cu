// Host launchers of the TF32 GEMM kernel and the CUDA-core fallback GEMM.
#include <mutex>

#include "gemm_tf32_pair.cuh"
#include "gemm_thin_rows.cuh"

namespace xtc {

// ---------------------------------------------------------------------------
// CUDA-core fp32 GEMM for shapes the TMA path cannot address (leading
// dimensions that are not a multiple of 4 elements) and for the FP32_SIMT
// precision mode.  64x64 tile, 16-deep, 4x4 micro-tile per thread.
// ---------------------------------------------------------------------------
template <bool A_T, bool B_T>
__global__ void __launch_bounds__(256)
gemm_f32_simt_kernel(const float* __restrict__ A, const float* __restrict__ B,
                     float* __restrict__ C, int M, int N, int K, int64_t lda, int64_t ldb,
                     int64_t ldc, int relu, float thr) {
  __shared__ float sA[16][64 + 4];
  __shared__ float sB[16][64 + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int mm, kk;
      if (!A_T) { kk = i & 15; mm = i >> 4; } else { mm = i & 63; kk = i >> 6; }
      int gm = m0 + mm, gk = k0 + kk;
      float v = 0.f;
      if (gm < M && gk < K) v = A_T ? A[static_cast<int64_t>(gk) * lda + gm]
                                    : A[static_cast<int64_t>(gm) * lda + gk];
      sA[kk][mm] = v;
    }
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      int nn, kk;
      if (!B_T) { nn = i & 63; kk = i >> 6; } else { kk = i & 15; nn = i >> 4; }
      int gn = n0 + nn, gk = k0 + kk;
      float v = 0.f;
      if (gn < N && gk < K) v = B_T ? B[static_cast<int64_t>(gn) * ldb + gk]
                                    : B[static_cast<int64_t>(gk) * ldb + gn];
      sB[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = sB[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn < N) {
        float v = acc[i][j];
        if (relu) v = fmaxf(v, thr);
        C[static_cast<int64_t>(gm) * ldc + gn] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Host launcher
// ---------------------------------------------------------------------------
namespace {

struct LaunchArgs {
  const float *A, *B, *Alo, *Blo;
  float* C;
  int64_t M, N, K, lda, ldb, ldc;
  bool a_t, b_t, relu;
  float thr;
  int stages;
  cudaStream_t stream;
  int* status = nullptr;  // status word to use instead of the per-device one
  int n_extra = 0;        // further copies of C to write (broadcast epilogue)
  float* extra[7] = {};
  float* mcast = nullptr;  // this rank's block of C through a multicast mapping (CTA-pair kernel)
  bool copier_warps = true;  // CTA-pair kernel: peers written by copier warps, not by the epilogue
  bool c_evict_first = true;  // CTA-pair kernel: L2 evict-first hint on the stores of C
  int split_k = 1;        // CTAs per output tile along K (needs partials + counters)
  float* partials = nullptr;
  int* counters = nullptr;
  bool cluster_k = false; // split-K reduced inside a thread-block cluster (no workspace)
  // CTA-pair kernel: zeroed workspace for the split tail (pair_tail_bytes), or NULL
  void* pair_tail = nullptr;
};

// Workspace of the pair kernel's split tail: at most `pairs` parked pieces, each
// with 8 flags and one 256 x tile_n raw accumulator.
size_t pair_tail_flag_bytes(int pairs) {
  return (static_cast<size_t>(pairs) * 8 * sizeof(int) + 255) & ~static_cast<size_t>(255);
}
size_t pair_tail_bytes(int pairs, int tile_n) {
  return pair_tail_flag_bytes(pairs) + static_cast<size_t>(pairs) * 256 * tile_n * sizeof(float);
}

template <int BN, int KSPANS, int A_MODE, bool B_MN, bool SPLIT3, bool TMA_STORE>
int launch_tc(const LaunchArgs& a) {
  using L = SmemLayout<BN, KSPANS, SPLIT3>;
  constexpr int BK = L::BK;
  constexpr bool A_MN = A_MODE == A_MNMAJOR;
  const int max_stages = L::max_stages(TMA_STORE);
  XTC_REQUIRE(max_stages >= 2, "gemm: tile %dx%dx%d does not fit shared memory", BM, BN, BK);
  int stages = a.stages <= 0 ? max_stages : a.stages;
  if (stages > max_stages) stages = max_stages;
  if (stages < 2) stages = 2;

  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));

  CUtensorMap tmA, tmB, tmAlo, tmBlo, tmC;
  memset(&tmAlo, 0, sizeof(tmAlo));
  memset(&tmBlo, 0, sizeof(tmBlo));
  memset(&tmC, 0, sizeof(tmC));
  int rc;
  auto mapA = [&](CUtensorMap* m, const float* p) {
    return A_MN ? make_tmap_2d(m, p, a.K, a.M, a.lda, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
                : make_tmap_2d(m, p, a.M, a.K, a.lda, 32, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  auto mapB = [&](CUtensorMap* m, const float* p) {
    return B_MN ? make_tmap_2d(m, p, a.K, a.N, a.ldb, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
                : make_tmap_2d(m, p, a.N, a.K, a.ldb, 32, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if ((rc = mapA(&tmA, a.A))) return rc;
  if ((rc = mapB(&tmB, a.B))) return rc;
  if (SPLIT3) {
    if ((rc = mapA(&tmAlo, a.Alo))) return rc;
    if ((rc = mapB(&tmBlo, a.Blo))) return rc;
  }
  if (TMA_STORE) {
    if ((rc = make_tmap_2d(&tmC, a.C, a.M, a.N, a.ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)))
      return rc;
  }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = a.C;
  p.ldc = a.ldc;
  p.M = static_cast<int>(a.M);
  p.N = static_cast<int>(a.N);
  p.K = static_cast<int>(a.K);
  p.tiles_m = static_cast<int>((a.M + BM - 1) / BM);
  p.tiles_n = static_cast<int>((a.N + BN - 1) / BN);
  p.k_blocks = static_cast<int>((a.K + BK - 1) / BK);
  // 3xTF32: hand the accumulator to the fp32 register sum every 256 elements of K
  p.chunk_kblocks = SPLIT3 ? (256 / BK) : p.k_blocks;
  p.relu = a.relu;
  p.relu_threshold = a.thr;
  p.status = a.status ? a.status : device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "gemm: device status word unavailable");
  p.n_extra = TMA_STORE ? a.n_extra : 0;
  for (int d = 0; d < p.n_extra; ++d) p.extra_dst[d] = a.extra[d];
  const bool in_cluster = !SPLIT3 && a.cluster_k && BN <= 128;
  const int want_split =
      SPLIT3 ? 1 : in_cluster ? cluster_pieces(p.k_blocks, a.split_k)
                              : (a.partials != nullptr && a.counters != nullptr) ? a.split_k : 1;
  p.split_kblocks = (p.k_blocks + want_split - 1) / want_split;
  p.split_k = (p.k_blocks + p.split_kblocks - 1) / p.split_kblocks;
  p.partials = a.partials;
  p.tile_counters = a.counters;
  if (p.split_k > 1) p.chunk_kblocks = p.split_kblocks;
  p.cluster_k = in_cluster && p.split_k >= 2 && p.split_k <= 8;
  XTC_REQUIRE(p.cluster_k || !in_cluster || p.split_k == 1,
              "gemm: the cluster split needs 2 to 8 pieces, got %d", p.split_k);

  auto kernel = gemm_tf32_kernel<BN, KSPANS, A_MODE, B_MN, SPLIT3, TMA_STORE>;
  const int smem = L::total(stages, TMA_STORE);
  static thread_local int configured_dev = -1;
  static thread_local int configured_smem = 0;
  if (configured_dev != dev || configured_smem < smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_dev = dev;
    configured_smem = smem;
  }
  const int tiles = p.tiles_m * p.tiles_n * p.split_k;
  // cluster split: one work item per CTA, the pieces of a tile in consecutive CTAs
  const int grid = p.cluster_k ? tiles : (tiles < sm_count(dev) ? tiles : sm_count(dev));
  p.group_n = panel_columns(sm_count(dev), BM, BN, p.tiles_n);
  XTC_CUDA_CHECK(launch_overlapped_clustered(kernel, grid, p.cluster_k ? p.split_k : 1, NUM_THREADS,
                                             smem, a.stream, tmA, tmB, tmAlo, tmBlo, tmC, p, stages));
  return XTC_CUDA_OK;
}

// CTA-pair kernel (tile rows 256): TF32 only, always with the TMA-store epilogue.
template <int BN, int KSPANS, bool A_MN, bool B_MN>
int launch_pair(const LaunchArgs& a) {
  using L = PairSmem<BN, KSPANS>;
  constexpr int BK = L::BK;
  const int max_stages = L::max_stages();
  int stages = a.stages <= 0 ? max_stages : a.stages;
  if (stages > max_stages) stages = max_stages;
  if (stages < 2) stages = 2;
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  CUtensorMap tmA, tmB, tmC;
  int rc;
  rc = A_MN ? make_tmap_2d(&tmA, a.A, a.K, a.M, a.lda, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
            : make_tmap_2d(&tmA, a.A, a.M, a.K, a.lda, 32, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = B_MN ? make_tmap_2d(&tmB, a.B, a.K, a.N, a.ldb, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)
            : make_tmap_2d(&tmB, a.B, a.N, a.K, a.ldb, 32, BN / 2, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if ((rc = make_tmap_2d(&tmC, a.C, a.M, a.N, a.ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = a.C;
  p.ldc = a.ldc;
  p.M = static_cast<int>(a.M);
  p.N = static_cast<int>(a.N);
  p.K = static_cast<int>(a.K);
  p.tiles_m = static_cast<int>((a.M + 2 * BM - 1) / (2 * BM));
  p.tiles_n = static_cast<int>((a.N + BN - 1) / BN);
  p.k_blocks = static_cast<int>((a.K + BK - 1) / BK);
  p.chunk_kblocks = p.k_blocks;
  p.relu = a.relu;
  p.relu_threshold = a.thr;
  p.status = a.status ? a.status : device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "gemm: device status word unavailable");
  p.n_extra = a.n_extra;
  for (int d = 0; d < p.n_extra; ++d) p.extra_dst[d] = a.extra[d];
  p.mc_dst = a.mcast;
  p.c_evict_first = a.n_extra == 0 && a.mcast == nullptr && a.c_evict_first;

  auto kernel = gemm_tf32_pair_kernel<BN, KSPANS, A_MN, B_MN>;
  const int smem = L::total(stages);
  static thread_local int configured_dev = -1;
  static thread_local int configured_smem = 0;
  static thread_local int max_pairs = 0;
  if (configured_dev != dev || configured_smem < smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    // how many 2-CTA clusters the device can hold at once with this footprint
    cudaLaunchConfig_t lc;
    memset(&lc, 0, sizeof(lc));
    lc.gridDim = dim3(static_cast<unsigned>(sm_count(dev) & ~1), 1, 1);
    lc.blockDim = dim3(NUM_THREADS, 1, 1);
    lc.dynamicSmemBytes = static_cast<size_t>(smem);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    lc.attrs = &attr;
    lc.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &lc) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count(dev) / 2;
    }
    max_pairs = n;
    configured_dev = dev;
    configured_smem = smem;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  p.group_n = panel_columns(pairs, 2 * BM, BN, p.tiles_n);
  // Split tail: the tiles of a last round that would leave at least half of the
  // pairs idle are cut along K, one piece per pair (see gemm_tf32_pair.cuh).  A problem of
  // fewer tiles than half the pairs (few rows, long K: 256 x 3072 x 8192 is 12 tiles) is
  // such a round as a whole.
  const int rem = tiles % pairs;
  const bool whole = tiles * 2 <= max_pairs;
  const int split = whole ? max_pairs / tiles : (rem > 0 ? pairs / rem : 0);
  // (each piece keeps at least 1024 of K: parking and re-reading a 256 x BN accumulator
  // costs more than a shorter piece saves)
  const int max_split = static_cast<int>(a.K / 1024);
  if (a.pair_tail != nullptr && (whole || tiles > pairs) && split >= 2 && max_split >= 2 &&
      max_pairs <= sm_count(dev) / 2) {
    p.tail_split = split < max_split ? split : max_split;
    if (p.tail_split > p.k_blocks) p.tail_split = p.k_blocks;
    p.tail_tiles = whole ? tiles : rem;
    p.tail_first = tiles - p.tail_tiles;
    p.sk_flags = static_cast<int*>(a.pair_tail);
    p.sk_partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a.pair_tail) +
                                             pair_tail_flag_bytes(sm_count(dev) / 2));
    if (p.tail_split < 2) p.tail_split = 0;
    else if (whole) pairs = tiles * p.tail_split;  // every piece on a pair of its own, all resident
  }
  const int threads =
      ((p.n_extra > 0 && a.copier_warps) || p.mc_dst != nullptr) ? PAIR_THREADS_BCAST : PAIR_THREADS;
  XTC_CUDA_CHECK(launch_overlapped(kernel, 2 * pairs, threads, smem, a.stream, tmA, tmB, tmC, p, stages));
  return XTC_CUDA_OK;
}

int dispatch_pair(const LaunchArgs& a, int tile_n, int tile_k) {
  const int ks = tile_k == 64 ? 2 : 1;
#define XTC_PAIR_CASE(BN_, KS_)                                                              \
  if (tile_n == BN_ && ks == KS_) {                                                          \
    if (!a.a_t && !a.b_t) return launch_pair<BN_, KS_, false, true>(a);                      \
    if (a.a_t && !a.b_t) return launch_pair<BN_, KS_, true, true>(a);                        \
    if (!a.a_t && a.b_t) return launch_pair<BN_, KS_, false, false>(a);                      \
    return launch_pair<BN_, KS_, true, false>(a);                                            \
  }
  XTC_PAIR_CASE(64, 1)
  XTC_PAIR_CASE(64, 2)
  XTC_PAIR_CASE(128, 1)
  XTC_PAIR_CASE(128, 2)
  XTC_PAIR_CASE(256, 1)
  XTC_PAIR_CASE(256, 2)
#undef XTC_PAIR_CASE
  set_error("gemm: unsupported tile_n=%d tile_k=%d for the CTA-pair kernel", tile_n, tile_k);
  return XTC_CUDA_ERR_UNSUPPORTED;
}

template <int BN, int KSPANS, bool SPLIT3, bool TMA_STORE>
int dispatch_major(const LaunchArgs& a) {
  // a_t: A stored [K,M] -> MN-major A.  b_t: B stored [N,K] -> K-major B.
  if (!a.a_t && !a.b_t) return launch_tc<BN, KSPANS, A_KMAJOR, true, SPLIT3, TMA_STORE>(a);
  if (a.a_t && !a.b_t) return launch_tc<BN, KSPANS, A_MNMAJOR, true, SPLIT3, TMA_STORE>(a);
  if (!a.a_t && a.b_t) return launch_tc<BN, KSPANS, A_KMAJOR, false, SPLIT3, TMA_STORE>(a);
  return launch_tc<BN, KSPANS, A_MNMAJOR, false, SPLIT3, TMA_STORE>(a);
}

template <bool SPLIT3, bool TMA_STORE>
int dispatch_tile(const LaunchArgs& a, int tile_n, int tile_k) {
  const int ks = tile_k == 64 ? 2 : 1;
  if (SPLIT3 && tile_n == 256) {
    // the epilogue keeps the running fp32 sum of a whole tile row in registers:
    // 128 columns per thread is the most that fits
    set_error("gemm: tile_n=256 is not available in 3xTF32 mode (use 64 or 128)");
    return XTC_CUDA_ERR_UNSUPPORTED;
  }
  switch (tile_n) {
    case 64:
      return ks == 1 ? dispatch_major<64, 1, SPLIT3, TMA_STORE>(a)
                     : dispatch_major<64, 2, SPLIT3, TMA_STORE>(a);
    case 128:
      return ks == 1 ? dispatch_major<128, 1, SPLIT3, TMA_STORE>(a)
                     : dispatch_major<128, 2, SPLIT3, TMA_STORE>(a);
    case 256:
      if constexpr (!SPLIT3) {
        return ks == 1 ? dispatch_major<256, 1, SPLIT3, TMA_STORE>(a)
                       : dispatch_major<256, 2, SPLIT3, TMA_STORE>(a);
      }
  }
  set_error("gemm: unsupported tile_n=%d tile_k=%d (tile_n in {64,128,256}, tile_k in {32,64})",
            tile_n, tile_k);
  return XTC_CUDA_ERR_UNSUPPORTED;
}

int launch_simt(const LaunchArgs& a) {
  dim3 grid(static_cast<unsigned>((a.N + 63) / 64), static_cast<unsigned>((a.M + 63) / 64));
  const int M = static_cast<int>(a.M), N = static_cast<int>(a.N), K = static_cast<int>(a.K);
  if (!a.a_t && !a.b_t)
    gemm_f32_simt_kernel<false, false><<<grid, 256, 0, a.stream>>>(a.A, a.B, a.C, M, N, K, a.lda, a.ldb, a.ldc, a.relu, a.thr);
  else if (a.a_t && !a.b_t)
    gemm_f32_simt_kernel<true, false><<<grid, 256, 0, a.stream>>>(a.A, a.B, a.C, M, N, K, a.lda, a.ldb, a.ldc, a.relu, a.thr);
  else if (!a.a_t && a.b_t)
    gemm_f32_simt_kernel<false, true><<<grid, 256, 0, a.stream>>>(a.A, a.B, a.C, M, N, K, a.lda, a.ldb, a.ldc, a.relu, a.thr);
  else
    gemm_f32_simt_kernel<true, true><<<grid, 256, 0, a.stream>>>(a.A, a.B, a.C, M, N, K, a.lda, a.ldb, a.ldc, a.relu, a.thr);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}

// A handful of rows (M <= 8): the matrix-vector kernel of gemm_thin_rows.cuh.
template <int MT>
int launch_thin_rows_mt(const LaunchArgs& a) {
  ThinRowsParams p;
  memset(&p, 0, sizeof(p));
  p.A = a.A; p.B = a.B; p.C = a.C;
  p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
  p.lda = a.lda; p.ldb = a.ldb; p.ldc = a.ldc;
  p.a_t = a.a_t; p.relu = a.relu; p.thr = a.thr;
  const size_t smem = thin_rows_smem(MT, a.K);
  // wide strips where there are enough of them to fill the chip (2 x 16384 x 4096: 49.2 us
  // against 55.7 us; 1 x 4096 x 9216 the other way round, 38.9 us against 27.3 us)
  const bool wide = a.N >= 8192;
  const int cols = wide ? THIN_COLS_WIDE : THIN_COLS;
  auto kernel = wide ? gemm_thin_rows_kernel<MT, THIN_COLS_WIDE> : gemm_thin_rows_kernel<MT, THIN_COLS>;
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  static thread_local int configured_dev[2] = {-1, -1};
  static thread_local size_t configured_smem[2] = {0, 0};
  if (configured_dev[wide] != dev || configured_smem[wide] < smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
    configured_dev[wide] = dev;
    configured_smem[wide] = smem;
  }
  const unsigned strips = static_cast<unsigned>((a.N + cols - 1) / cols);
  XTC_CUDA_CHECK(launch_overlapped_clustered(kernel, strips * THIN_KSPLIT, THIN_KSPLIT, THIN_THREADS,
                                             smem, a.stream, p));
  return XTC_CUDA_OK;
}
int thin_rows_mt(int64_t M) { return M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8)); }
int launch_thin_rows(const LaunchArgs& a) {
  switch (thin_rows_mt(a.M)) {
    case 1: return launch_thin_rows_mt<1>(a);
    case 2: return launch_thin_rows_mt<2>(a);
    case 4: return launch_thin_rows_mt<4>(a);
    default: return launch_thin_rows_mt<8>(a);
  }
}

bool tma_addressable(const void* p, int64_t ld) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld % 4) == 0;
}

size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

}  // namespace

// Default CTA tile for a problem: the widest N tile that still yields at least
// one tile per SM, else the narrower ones (more tiles for small problems).
static int default_tile_n(int64_t M, int64_t N, int sms) {
  const int64_t tm = (M + BM - 1) / BM;
  for (int bn : {256, 128, 64}) {
    if (N >= bn && tm * ((N + bn - 1) / bn) >= sms) return bn;
  }
  if (N <= 64) return 64;
  if (N <= 128) return 128;
  return tm * ((N + 127) / 128) >= sms / 2 ? 128 : 64;
}

// How many clusters of `size` CTAs of the single-CTA GEMM kernel the device runs at once
// (the kernel takes a whole SM, and a cluster must sit inside one GPC).  Asked of the
// runtime once per device and size; a split whose clusters do not all fit runs in waves
// and loses what it was meant to gain.
int cluster_capacity(int dev, int size) {
  if (size <= 1) return sm_count(dev);
  static std::mutex mu;
  static int cache[16][9];  // 0 = not asked yet
  if (dev < 0 || dev >= 16 || size > 8) return sm_count(dev) / (size * 2);
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev][size] == 0) {
    using L = SmemLayout<64, 2, false>;
    auto kernel = gemm_tf32_kernel<64, 2, A_KMAJOR, true, false, false>;
    const int smem = L::total(L::max_stages(false), false);
    int n = 0;
    cudaLaunchConfig_t lc;
    memset(&lc, 0, sizeof(lc));
    lc.gridDim = dim3(static_cast<unsigned>(size) * 64u, 1, 1);
    lc.blockDim = dim3(NUM_THREADS, 1, 1);
    lc.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    memset(&attr, 0, sizeof(attr));
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(size);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    lc.attrs = &attr;
    lc.numAttrs = 1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kernel, &lc) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count(dev) / (size * 2);  // a guess on the safe side
    }
    cache[dev][size] = n;
  }
  return cache[dev][size];
}

// Kernel and tile for a TF32 problem whose caller named nothing (all of tile_m, tile_n,
// tile_k, split_k zero): the candidate with the smallest modelled time.  The model is the
// shared-memory / tensor-pipe cost of one K step of 8 per tile (measured: 128 clocks for a
// 256x256 pair tile, 128 for 128x128, 192 for 128x256, 96 for 256x128 and 128x64), times
// the K steps, times the rounds of tiles over the SMs (the split tail of the pair kernel
// shortens a last round that is at most half full), plus a fixed 6 us; single-CTA
// candidates with few tiles may split K.  Tiles up to 128 columns wide split into 2 to 8
// pieces inside a thread-block cluster while all clusters fit on the device at once
// (`cluster_cap[s]`, NULL = no cluster split): 1 us + 1 us per 64 tile columns + 0.25 us per
// piece for the reduction through distributed shared memory (512x256x1024: 10.1 us
// unsplit, 7.9 us in 4 pieces, 8.2 us in 6; 256x256x4096: 29.1 us unsplit, 9.9 us in 8
// pieces; 512x512x8192: 23.5 us in 4 pieces, 19.5 us in 6).
// Other splits go through a workspace (`split_ok`), which costs 3 us + 1.15 us per piece
// for the reduction pass.
AutoChoice choose_tf32_default(int64_t M, int64_t N, int64_t K, int sms, bool pair_ok,
                               bool split_ok, const int* cluster_cap, bool pair_tail_ok) {
  struct Cand { int tm, tn; double clk; };
  // on a tie the earlier candidate wins: one CTA per tile before CTA pairs
  static const Cand cands[] = {{128, 64, 96.0}, {128, 128, 128.0}, {128, 256, 192.0},
                               {256, 128, 96.0}, {256, 256, 128.0}};
  const double clk_per_us = 1900.0, fixed = 6.0 * clk_per_us;
  const double ksteps = static_cast<double>((K + 7) / 8);
  AutoChoice best{128, 128, 32, 1};
  double best_t = 1e300;
  // Short K under a narrow N (1x1 convolutions as GEMMs): a tile is one or two K stages, the
  // step is the epilogue and HBM, and the per-tile hand-offs of a CTA pair only cost
  // (100352x256x64: 33 us with pairs, 26 us with 128x256 tiles, at the HBM floor of 20 us;
  // 100352x64x256: 29 - 31 us against 24 us).
  const bool skinny = K <= 256;
  // Few rows and a long K (a handful of token rows against a weight matrix): the step streams B
  // from HBM once and no tile order gives the operands any reuse, so the cost model below, which
  // counts tensor clocks, does not rank the shapes.  Measured instead (B200, us, M x N x K):
  //   256 x 3072 x 8192: pairs 256x128 35.4 | pairs 256x256 49.9 | 128x128 in 2 pieces 45.1
  //   256 x 8192 x 3072: pairs 256x128 29.2 | pairs 256x256 37.9 | 128x128 32.4
  //   256 x 2048 x 8192: 128x128 in 4 pieces 24.5 | pairs 256x128 30.1
  //   128 x 4096 x 8192: 128x128 in 4 pieces 29.4;  128 x 8192 x 4096: 128x64 31.7, 128x128 in 2 33.0
  if (M <= 256 && K >= 2048 && N >= 1024) {
    if (pair_ok && pair_tail_ok && M > 128 && N >= 3072)
      return {256, 128, 64, 1};  // the pair kernel cuts K itself
    const int64_t tiles = ((M + 127) / 128) * ((N + 127) / 128);
    int split = 1;
    if (cluster_cap != nullptr && N % 4 == 0) {
      // the most pieces that leave every cluster resident and 768 of K to a piece
      // (169 x 1024 x 4608: 16.9 us in 4 pieces, 14.9 us in 6; 289 x 1024 x 9216: 25.8 us in 4, 23.0 in 5)
      const int kblocks = static_cast<int>((K + 63) / 64);
      for (int s = 2; s <= 8 && tiles * s <= sms && K / s >= 768; ++s)
        if (tiles <= cluster_cap[s] && cluster_pieces(kblocks, s) == s) split = s;
    }
    return {128, 128, 64, split};
  }
  for (const Cand& c : cands) {
    if (c.tm == 256 && (!pair_ok || skinny)) continue;
    const int64_t tiles = ((M + c.tm - 1) / c.tm) * ((N + c.tn - 1) / c.tn);
    const int64_t slots = c.tm == 256 ? sms / 2 : sms;
    const int64_t full = tiles / slots, rem = tiles % slots;
    double rounds = static_cast<double>(full);
    double tail_cost = 0.0;
    if (rem) {
      // the pair kernel cuts a last (or only) round that fills at most half of the pairs along
      // K, at least 1024 per piece; one pair sums the parked pieces of a tile, about 2.3 us per
      // piece of 256 x 256
      int64_t pieces = (c.tm == 256 && split_ok && pair_tail_ok && rem * 2 <= slots) ? slots / rem : 1;
      if (pieces > K / 1024) pieces = K / 1024;
      if (pieces >= 2) {
        rounds += 1.0 / static_cast<double>(pieces);
        tail_cost = (1.0 + 2.3 * static_cast<double>(pieces) * c.tn / 256.0) * clk_per_us;
      } else {
        rounds += 1.0;
      }
    }
    // K per stage: 64 halves the barrier traffic (2048 x 256 x 2048 on 128 x 128 tiles in 4
    // pieces: 11.9 us against 13.3 us); 256 x 256 pair tiles on few rows of tiles get
    // 32 (six stages instead of three hide the HBM latency: 512 x 4096 x 8192 61.8 us against
    // 68.2 us, 1024 x 4096 x 4096 53.0 us against 54.7 us)
    const int tile_k = c.tm == 256 ? (K >= 128 && !(c.tn == 256 && M <= 1024) ? 64 : 32)
                                   : ((c.tn <= 128 || skinny) && K >= 128 ? 64 : 32);
    double t = rounds * ksteps * c.clk + fixed + tail_cost;
    int split = 1;
    const int64_t kblocks = (K + tile_k - 1) / tile_k;
    if (cluster_cap != nullptr && c.tm == 128 && c.tn <= 128 && N % 4 == 0) {
      for (int s = 2; s <= 8 && tiles <= cluster_cap[s] && tiles * s <= slots && s <= kblocks; ++s) {
        if (cluster_pieces(static_cast<int>(kblocks), s) != s) continue;  // an empty last piece
        // the longest piece sets the pace: ceil(kblocks / s) stages of tile_k
        const double piece_steps = static_cast<double>((kblocks + s - 1) / s) * (tile_k / 8);
        const double ts = piece_steps * c.clk + fixed + (1.0 + c.tn / 64.0 + 0.25 * s) * clk_per_us;
        if (ts < t) { t = ts; split = s; }
      }
    }
    if (split == 1 && split_ok && c.tm == 128 && tiles * 2 <= slots) {
      for (int s = 2; s <= 16 && tiles * s <= slots && s <= kblocks; s *= 2) {
        // the reducing CTA reads s partial tiles of 128 x tn floats (calibrated at tn = 64)
        const double ts = ksteps * c.clk / s + fixed + (3.0 + 1.15 * s * (c.tn / 64.0)) * clk_per_us;
        if (ts < t) { t = ts; split = s; }
      }
    }
    if (t < best_t) {
      best_t = t;
      best = {c.tm, c.tn, tile_k, split};
    }
  }
  return best;
}
static bool is_full_auto(const xtc_cuda_gemm_config& c) {
  return c.precision == XTC_CUDA_PRECISION_TF32 && c.tile_m == 0 && c.tile_n == 0 && c.tile_k == 0 &&
         c.split_k == 0;
}

// What the single-CTA TF32 kernel will run with for a problem and a request:
// tile shape and the split-K factor (1 = none).  Used by the launcher and by the
// workspace query so that both agree.
struct TfShape {
  int tile_n, tile_k, split_k, tiles;
};
static TfShape resolve_tf32_shape(int64_t M, int64_t N, int64_t K, const xtc_cuda_gemm_config& c,
                                  int sms) {
  TfShape s;
  s.tile_n = c.tile_n ? c.tile_n : default_tile_n(M, N, sms);
  s.tile_k = c.tile_k ? c.tile_k : 32;
  if (s.tile_n != 64 && s.tile_n != 128 && s.tile_n != 256) s.tile_n = 128;  // rejected later
  if (s.tile_k != 32 && s.tile_k != 64) s.tile_k = 32;
  s.tiles = static_cast<int>(((M + BM - 1) / BM) * ((N + s.tile_n - 1) / s.tile_n));
  const int k_blocks = static_cast<int>((K + s.tile_k - 1) / s.tile_k);
  int want = c.split_k;
  // 0 (auto) currently means off: measured on 512x1024x256, the extra pass over the
  // partial tiles (one SM reads split_k tiles from L2 at ~100 GB/s) costs more than
  // the idle SMs would have gained (10.7 us unsplit, 13.4 us at 2, 19.7 us at 8).
  if (want == 0) want = 1;
  (void)sms;
  if (want > k_blocks) want = k_blocks;
  if (want < 1 || c.precision != XTC_CUDA_PRECISION_TF32) want = 1;
  // no empty splits: recompute the count from the per-split length
  const int per = (k_blocks + want - 1) / want;
  s.split_k = (k_blocks + per - 1) / per;
  return s;
}

}  // namespace xtc

using namespace xtc;

extern "C" int xtc_cuda_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int flags,
                                             const xtc_cuda_gemm_config* cfg, size_t* bytes) {
  XTC_REQUIRE(bytes != nullptr, "gemm_workspace_bytes: bytes is NULL");
  XTC_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_workspace_bytes: empty problem");
  (void)flags;
  *bytes = 0;
  xtc_cuda_gemm_config c;
  memset(&c, 0, sizeof(c));
  if (cfg) c = *cfg;
  if (c.precision == XTC_CUDA_PRECISION_3XTF32) {
    // hi and lo parts of both operands, each a dense copy
    *bytes = 2 * align256(static_cast<size_t>(M) * K * 4) + 2 * align256(static_cast<size_t>(K) * N * 4);
    return XTC_CUDA_OK;
  }
  int dev = 0;
  int sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) sms = sm_count(dev); else cudaGetLastError();
  if (is_full_auto(c)) {  // size for what the library would pick itself (see gemm_impl)
    int caps[9] = {};
    for (int sz = 2; sz <= 8; ++sz) caps[sz] = cluster_capacity(dev, sz);
    const AutoChoice pick = choose_tf32_default(M, N, K, sms, true, true, caps);
    c.tile_m = pick.tile_m;
    c.tile_n = pick.tile_n;
    c.tile_k = pick.tile_k;
    c.split_k = pick.tile_m == 2 * BM ? 0 : pick.split_k;
  }
  if (c.precision == XTC_CUDA_PRECISION_TF32 && c.tile_m == 2 * BM && c.split_k != 1) {
    // the CTA-pair kernel's split tail (split_k = 1 turns it off)
    *bytes = pair_tail_bytes(sms / 2, c.tile_n ? c.tile_n : 256);
    return XTC_CUDA_OK;
  }
  if (c.precision == XTC_CUDA_PRECISION_TF32 && c.tile_m != 2 * BM) {
    const TfShape s = resolve_tf32_shape(M, N, K, c, sms);
    // a split the launcher reduces inside a cluster needs nothing (assuming, as the launcher
    // checks, a 16-byte aligned C with a pitch that is a multiple of 4)
    const bool in_cluster = c.variant != 1 && s.split_k >= 2 && s.split_k <= 8 &&
                            s.tile_n <= 128 && N % 4 == 0 && s.tiles <= cluster_capacity(dev, s.split_k);
    if (s.split_k > 1 && !in_cluster)  // tile counters, then the partial tiles [split][tile][128][tile_n]
      *bytes = align256(static_cast<size_t>(s.tiles) * 4) +
               static_cast<size_t>(s.split_k) * s.tiles * BM * s.tile_n * 4;
  }
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_gemm_default_config(int64_t M, int64_t N, int64_t K, xtc_cuda_gemm_config* out) {
  XTC_REQUIRE(out != nullptr, "gemm_default_config: out is NULL");
  XTC_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_default_config: empty problem");
  memset(out, 0, sizeof(*out));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) sms = sm_count(dev); else cudaGetLastError();
  int caps[9] = {};
  for (int sz = 2; sz <= 8; ++sz) caps[sz] = cluster_capacity(dev, sz);
  const AutoChoice pick = choose_tf32_default(M, N, K, sms, true, true, caps);
  out->tile_m = pick.tile_m;
  out->tile_n = pick.tile_n;
  out->tile_k = pick.tile_k;
  out->split_k = pick.tile_m == 2 * BM ? 0 : pick.split_k;
  out->epilogue = 2;
  return XTC_CUDA_OK;
}

static int gemm_impl(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                     int64_t lda, int64_t ldb, int64_t ldc, int flags, float relu_threshold,
                     const xtc_cuda_gemm_config* cfg, void* workspace, size_t workspace_bytes,
                     void* stream, int n_extra, float* const* extra, float* mcast = nullptr) {
  XTC_REQUIRE(A && B && C, "gemm: NULL operand");
  XTC_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem %lldx%lldx%lld", (long long)M,
              (long long)N, (long long)K);
  XTC_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "gemm: dimension too large");
  const bool a_t = flags & XTC_CUDA_GEMM_A_TRANSPOSED;
  const bool b_t = flags & XTC_CUDA_GEMM_B_TRANSPOSED;
  XTC_REQUIRE(lda >= (a_t ? M : K), "gemm: lda=%lld too small", (long long)lda);
  XTC_REQUIRE(ldb >= (b_t ? K : N), "gemm: ldb=%lld too small", (long long)ldb);
  XTC_REQUIRE(ldc >= N, "gemm: ldc=%lld too small", (long long)ldc);

  xtc_cuda_gemm_config c;
  memset(&c, 0, sizeof(c));
  if (cfg) c = *cfg;
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));

  LaunchArgs a;
  a.A = A; a.B = B; a.Alo = nullptr; a.Blo = nullptr; a.C = C;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldb = ldb; a.ldc = ldc;
  a.a_t = a_t; a.b_t = b_t;
  a.relu = flags & XTC_CUDA_FUSE_RELU;
  a.thr = relu_threshold;
  a.stages = c.stages;
  a.stream = static_cast<cudaStream_t>(stream);
  a.c_evict_first = c.variant != 2;

  const bool tma_ok = tma_addressable(A, lda) && tma_addressable(B, ldb);
  if (n_extra > 0) {
    XTC_REQUIRE(n_extra <= 7 && extra != nullptr, "gemm_bcast: at most 7 extra destinations");
    XTC_REQUIRE(tma_ok && tma_addressable(C, ldc) && c.precision != XTC_CUDA_PRECISION_FP32_SIMT,
                "gemm_bcast: operands and C must be 16-byte aligned with pitches that are multiples of 4");
    a.n_extra = n_extra;
    a.copier_warps = c.variant != 1;
    for (int d = 0; d < n_extra; ++d) {
      XTC_REQUIRE(tma_addressable(extra[d], ldc), "gemm_bcast: destination %d is NULL or misaligned", d);
      a.extra[d] = extra[d];
    }
  }
  if (mcast != nullptr) {
    XTC_REQUIRE(tma_ok && tma_addressable(C, ldc) && tma_addressable(mcast, ldc) &&
                    c.precision == XTC_CUDA_PRECISION_TF32,
                "gemm_mcast: TF32 only; operands, C and the multicast address must be 16-byte aligned "
                "with pitches that are multiples of 4");
    XTC_REQUIRE(c.tile_m == 0 || c.tile_m == 2 * BM,
                "gemm_mcast: the multicast stores are issued by the CTA-pair kernel (tile_m = 256)");
    c.tile_m = 2 * BM;
    a.mcast = mcast;
  }
  // Nothing named by the caller: the library picks kernel, tile and split itself.
  const bool full_auto = is_full_auto(c);
  // at most 8 rows: a matrix-vector product per row, bound by reading B once
  if (full_auto && M <= 8 && !b_t && n_extra == 0 && mcast == nullptr && N % 4 == 0 &&
      tma_addressable(B, ldb) && tma_addressable(C, ldc) &&
      thin_rows_smem(thin_rows_mt(M), K) <= 200 * 1024 && (N + THIN_COLS - 1) / THIN_COLS <= 65535)
    return launch_thin_rows(a);
  if (c.precision == XTC_CUDA_PRECISION_FP32_SIMT || !tma_ok) return launch_simt(a);

  if (full_auto) {
    int caps[9] = {};
    for (int sz = 2; sz <= 8; ++sz) caps[sz] = cluster_capacity(dev, sz);
    const AutoChoice pick = choose_tf32_default(M, N, K, sm_count(dev), tma_addressable(C, ldc), true,
                                                tma_addressable(C, ldc) && n_extra == 0 ? caps : nullptr);
    c.tile_m = pick.tile_m;
    c.tile_n = pick.tile_n;
    c.tile_k = pick.tile_k;
    c.split_k = pick.tile_m == 2 * BM ? 0 : pick.split_k;
    // bulk tensor stores for the one-CTA kernel too: with one or two K stages per tile the
    // epilogue is the step, and direct stores take 39 us where TMA stores take 26
    if (pick.tile_m == BM && c.epilogue == 0 && tma_addressable(C, ldc)) c.epilogue = 2;
  }
  XTC_REQUIRE(c.tile_m == 0 || c.tile_m == BM || c.tile_m == 2 * BM,
              "gemm: tile_m=%d unsupported (128, or 256 for the CTA-pair kernel)", c.tile_m);
  if (c.tile_m == 2 * BM) {
    XTC_REQUIRE(c.precision == XTC_CUDA_PRECISION_TF32, "gemm: tile_m=256 is a TF32-only configuration");
    XTC_REQUIRE(tma_addressable(C, ldc), "gemm: tile_m=256 needs a 16-byte aligned C with ldc %% 4 == 0");
    const int tn = c.tile_n ? c.tile_n : 256;
    // the split tail is an optimisation: without a (zeroed) workspace the tiles go round-robin
    if (c.split_k != 1 && workspace != nullptr &&
        workspace_bytes >= pair_tail_bytes(sm_count(dev) / 2, tn))
      a.pair_tail = workspace;
    return dispatch_pair(a, tn, c.tile_k ? c.tile_k : 32);
  }
  const TfShape shp = resolve_tf32_shape(M, N, K, c, sm_count(dev));
  int tile_n = c.tile_n ? c.tile_n : shp.tile_n;
  if (c.precision == XTC_CUDA_PRECISION_3XTF32 && c.tile_n == 0 && tile_n > 128) tile_n = 128;
  const int tile_k = c.tile_k ? c.tile_k : 32;
  // 2 to 8 pieces of tiles up to 128 columns wide are reduced inside a thread-block cluster
  // (variant = 1 keeps the workspace form)
  const bool cluster_split = shp.split_k > 1 && n_extra == 0 && c.variant != 1 &&
                             shp.split_k >= 2 && shp.split_k <= 8 &&
                             shp.tile_n <= 128 && tma_addressable(C, ldc) && N % 4 == 0 &&
                             c.precision == XTC_CUDA_PRECISION_TF32 &&
                             shp.tiles <= cluster_capacity(dev, shp.split_k);
  if (cluster_split) {
    a.split_k = shp.split_k;
    a.cluster_k = true;
  } else if (shp.split_k > 1 && n_extra == 0) {
    const size_t counters = align256(static_cast<size_t>(shp.tiles) * 4);
    const size_t need = counters + static_cast<size_t>(shp.split_k) * shp.tiles * BM * shp.tile_n * 4;
    if (workspace != nullptr && workspace_bytes >= need) {
      a.split_k = shp.split_k;
      a.counters = static_cast<int*>(workspace);
      a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + counters);
    } else {
      // automatic split-K is an optimisation: without a workspace run unsplit
      XTC_REQUIRE(full_auto || c.split_k == 0,
                  "gemm: split_k=%d needs %zu bytes of zeroed workspace, got %zu", c.split_k, need,
                  workspace ? workspace_bytes : static_cast<size_t>(0));
    }
  }
  // the broadcast epilogue reads the tile back from the store staging buffers
  const bool tma_store = (c.epilogue == 2 || n_extra > 0) && tma_addressable(C, ldc);

  if (c.precision == XTC_CUDA_PRECISION_3XTF32) {
    size_t need = 0;
    xtc_cuda_gemm_workspace_bytes(M, N, K, flags, &c, &need);
    XTC_REQUIRE(workspace != nullptr && workspace_bytes >= need,
                "gemm: 3xTF32 needs %zu bytes of workspace, got %zu", need, workspace_bytes);
    XTC_REQUIRE(lda == (a_t ? M : K) && ldb == (b_t ? K : N),
                "gemm: 3xTF32 requires dense operands");
    uint8_t* w = static_cast<uint8_t*>(workspace);
    float* Ahi = reinterpret_cast<float*>(w);
    float* Alo = reinterpret_cast<float*>(w + align256(static_cast<size_t>(M) * K * 4));
    float* Bhi = reinterpret_cast<float*>(w + 2 * align256(static_cast<size_t>(M) * K * 4));
    float* Blo = reinterpret_cast<float*>(w + 2 * align256(static_cast<size_t>(M) * K * 4) +
                                          align256(static_cast<size_t>(K) * N * 4));
    int rc;
    if ((rc = xtc_cuda_split_tf32(A, Ahi, Alo, M * K, stream))) return rc;
    if ((rc = xtc_cuda_split_tf32(B, Bhi, Blo, K * N, stream))) return rc;
    a.A = Ahi; a.Alo = Alo; a.B = Bhi; a.Blo = Blo;
    return tma_store ? dispatch_tile<true, true>(a, tile_n, tile_k)
                     : dispatch_tile<true, false>(a, tile_n, tile_k);
  }
  XTC_REQUIRE(c.precision == XTC_CUDA_PRECISION_TF32, "gemm: unknown precision %d", c.precision);
  return tma_store ? dispatch_tile<false, true>(a, tile_n, tile_k)
                   : dispatch_tile<false, false>(a, tile_n, tile_k);
}

extern "C" int xtc_cuda_gemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t N,
                                 int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int flags,
                                 float relu_threshold, const xtc_cuda_gemm_config* cfg,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, flags, relu_threshold, cfg, workspace,
                   workspace_bytes, stream, 0, nullptr);
}

extern "C" int xtc_cuda_gemm_f32_bcast(const float* A, const float* B, float* C,
                                       float* const* extra_dst, int n_extra, int64_t M, int64_t N,
                                       int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int flags,
                                       float relu_threshold, const xtc_cuda_gemm_config* cfg,
                                       void* workspace, size_t workspace_bytes, void* stream) {
  XTC_REQUIRE(n_extra >= 0, "gemm_bcast: negative destination count");
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, flags, relu_threshold, cfg, workspace,
                   workspace_bytes, stream, n_extra, extra_dst);
}

extern "C" int xtc_cuda_gemm_f32_mcast(const float* A, const float* B, float* C, float* mcast_C,
                                       int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                       int64_t ldc, int flags, float relu_threshold,
                                       const xtc_cuda_gemm_config* cfg, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  XTC_REQUIRE(mcast_C != nullptr, "gemm_mcast: NULL multicast address");
  return gemm_impl(A, B, C, M, N, K, lda, ldb, ldc, flags, relu_threshold, cfg, workspace,
                   workspace_bytes, stream, 0, nullptr, mcast_C);
}

// Exporting device memory to the other processes of the box (one process per GPU)
// so that their GEMMs can store into it.
extern "C" int xtc_cuda_ipc_export(void* device_ptr, void* handle64) {
  XTC_REQUIRE(device_ptr && handle64, "ipc_export: NULL argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  XTC_CUDA_CHECK(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle64, &h, 64);
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_ipc_import(const void* handle64, void** device_ptr) {
  XTC_REQUIRE(device_ptr && handle64, "ipc_import: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  *device_ptr = nullptr;
  XTC_CUDA_CHECK(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return XTC_CUDA_OK;
}
extern "C" int xtc_cuda_ipc_release(void* device_ptr) {
  if (device_ptr) XTC_CUDA_CHECK(cudaIpcCloseMemHandle(device_ptr));
  return XTC_CUDA_OK;
}

// ---------------------------------------------------------------------------
// 3xTF32 GEMM that allocates nothing
// ---------------------------------------------------------------------------
namespace {
// Scratch for the hi/lo operand split, resident in every GPU that loads the
// library until the process exits.
constexpr size_t NOALLOC_SCRATCH_BYTES = 32u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
static __device__ __align__(256) int g_noalloc_status[64];

struct NoallocDevice {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device addresses, resolved once per device
  int* status = nullptr;
};
std::mutex g_noalloc_mutex;
NoallocDevice g_noalloc[64];
}  // namespace

int xtc::noalloc_status_fetch_and_clear(int dev, int* status) {
  *status = 0;
  if (dev < 0 || dev >= 64) return XTC_CUDA_OK;
  int* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc[dev].ready) word = g_noalloc[dev].status;
  }
  if (word == nullptr) return XTC_CUDA_OK;  // the entry point has not run on this device
  XTC_CUDA_CHECK(cudaMemcpy(status, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status != 0) XTC_CUDA_CHECK(cudaMemset(word, 0, sizeof(int)));
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_gemm_f32_3xtf32_noalloc(const float* A, const float* B, float* C,
                                                int64_t M, int64_t N, int64_t K, int flags,
                                                float relu_threshold, void* stream) {
  XTC_REQUIRE(A && B && C, "gemm_noalloc: NULL operand");
  XTC_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_noalloc: empty problem");
  XTC_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), "gemm_noalloc: dimension too large");
  const bool a_t = flags & XTC_CUDA_GEMM_A_TRANSPOSED;
  const bool b_t = flags & XTC_CUDA_GEMM_B_TRANSPOSED;
  const int64_t lda = a_t ? M : K, ldb = b_t ? K : N, ldc = N;
  XTC_REQUIRE(tma_addressable(A, lda) && tma_addressable(B, ldb) && tma_addressable(C, ldc),
              "gemm_noalloc: A, B and C must be 16-byte aligned with row lengths that are multiples of 4");
  // Bound the element counts before any byte arithmetic: with M, N, K up to 2^31 the
  // products below would wrap in size_t and pass the size check.
  constexpr int64_t MAX_ELEMS = static_cast<int64_t>(NOALLOC_SCRATCH_BYTES / 8);  // hi + lo, 4 bytes each
  const bool fits = M <= MAX_ELEMS / K && K <= MAX_ELEMS / N;  // M*K and K*N each within the scratch
  const size_t a_bytes = fits ? align256(static_cast<size_t>(M) * K * 4) : 0;
  const size_t b_bytes = fits ? align256(static_cast<size_t>(K) * N * 4) : 0;
  const size_t need = 2 * a_bytes + 2 * b_bytes;
  XTC_REQUIRE(fits && need <= NOALLOC_SCRATCH_BYTES,
              "gemm_noalloc: A (%lld x %lld) and B (%lld x %lld) need %.0f bytes of scratch for the "
              "operand split, the built-in scratch holds %zu (use xtc_cuda_gemm_f32 with a caller "
              "workspace for larger problems)",
              (long long)M, (long long)K, (long long)K, (long long)N,
              8.0 * (static_cast<double>(M) * K + static_cast<double>(K) * N), NOALLOC_SCRATCH_BYTES);
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  XTC_REQUIRE(dev >= 0 && dev < 64, "gemm_noalloc: device ordinal %d out of range", dev);
  NoallocDevice nd;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc[dev].ready) {
      // In host code the array names are only handles: the addresses the kernels
      // need come from the runtime, once per device, with that device current.
      void* p = nullptr;
      XTC_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
      g_noalloc[dev].scratch = static_cast<unsigned char*>(p);
      XTC_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_status));
      g_noalloc[dev].status = static_cast<int*>(p);
      g_noalloc[dev].ready = true;
    }
    nd = g_noalloc[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* Ahi = reinterpret_cast<float*>(nd.scratch);
  float* Alo = reinterpret_cast<float*>(nd.scratch + a_bytes);
  float* Bhi = reinterpret_cast<float*>(nd.scratch + 2 * a_bytes);
  float* Blo = reinterpret_cast<float*>(nd.scratch + 2 * a_bytes + b_bytes);
  // Every byte of the scratch that the GEMM reads is rewritten by the two split
  // kernels below, so nothing left by an earlier call has to be cleared.
  int rc;
  if ((rc = xtc_cuda_split_tf32(A, Ahi, Alo, M * K, stream))) return rc;
  if ((rc = xtc_cuda_split_tf32(B, Bhi, Blo, K * N, stream))) return rc;
  LaunchArgs a;
  a.A = Ahi; a.Alo = Alo; a.B = Bhi; a.Blo = Blo; a.C = C;
  a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldb = ldb; a.ldc = ldc;
  a.a_t = a_t; a.b_t = b_t;
  a.relu = flags & XTC_CUDA_FUSE_RELU;
  a.thr = relu_threshold;
  a.stages = 0;
  a.stream = s;
  a.status = nd.status;
  const int tile_n = N <= 64 ? 64 : 128;
  return dispatch_tile<true, false>(a, tile_n, 32);
}
