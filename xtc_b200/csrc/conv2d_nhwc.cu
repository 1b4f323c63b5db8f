// NHWC x HWIO convolution as an implicit GEMM on the TF32 tensor cores:
//   M = B*OH*OW output pixels, N = F output channels, K = R*S*C.
// The A operand is never materialised: the producer warp of the GEMM kernel
// fetches [128 pixels x 32 channels] slabs with im2col-mode TMA, one filter
// tap (r, s) at a time.  Zero padding of H and W is folded into the fetch (the
// tensor map's bounding box starts at -pad and out-of-bounds reads return 0),
// relu into the epilogue.  Shapes TMA cannot address (C or F not a multiple of
// 4) run on a direct CUDA-core kernel.
#include "conv2d_halo_pair.cuh"
#include "conv2d_halo_taps.cuh"
#include "conv2d_halo_slide.cuh"
#include "conv2d_halo_stream.cuh"
#include "gemm_tf32_pair.cuh"

#ifdef XTC_TRACE
extern "C" int xtc_cuda_debug_set_halo_trace(long long* buffer) {
  return cudaMemcpyToSymbol(xtc::g_halo_trace, &buffer, sizeof(buffer)) == cudaSuccess ? 0 : 2;
}
#endif

namespace xtc {

struct ConvArgs {
  const float *X, *Wt;
  float* Y;
  int64_t B, H, W, C, R, S, F;
  int sh, sw, pt, pb, pl, pr;
  int64_t OH, OW;
  bool relu;
  float thr;
  int stages;
  cudaStream_t stream;
  int split_k = 1;            // im2col kernel, one CTA per tile: CTAs sharing a tile along K
  float* partials = nullptr;  // [split][tile][128][tile_n]
  int* counters = nullptr;    // [tile], zeroed once
  bool cluster_k = false;     // 2 to 8 pieces summed inside a thread-block cluster (no workspace)
};

__global__ void __launch_bounds__(256)
conv2d_direct_kernel(const float* __restrict__ X, const float* __restrict__ Wt,
                     float* __restrict__ Y, int64_t total, int H, int W, int C, int R, int S,
                     int F, int OH, int OW, int sh, int sw, int pt, int pl, int relu, float thr) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += stride) {
    const int f = static_cast<int>(i % F);
    int64_t pix = i / F;
    const int ow = static_cast<int>(pix % OW); pix /= OW;
    const int oh = static_cast<int>(pix % OH);
    const int64_t b = pix / OH;
    float acc = 0.f;
    for (int r = 0; r < R; ++r) {
      const int ih = oh * sh - pt + r;
      if (ih < 0 || ih >= H) continue;
      for (int s = 0; s < S; ++s) {
        const int iw = ow * sw - pl + s;
        if (iw < 0 || iw >= W) continue;
        const float* xp = X + ((b * H + ih) * W + iw) * C;
        const float* wp = Wt + (static_cast<int64_t>(r) * S + s) * C * F + f;
        for (int c = 0; c < C; ++c) acc = fmaf(xp[c], wp[static_cast<int64_t>(c) * F], acc);
      }
    }
    if (relu) acc = fmaxf(acc, thr);
    Y[i] = acc;
  }
}

// ---------------------------------------------------------------------------
// Thin inputs (a few channels: the first layer of an image network)
// ---------------------------------------------------------------------------
// With C channels the tensor-core kernels spend a K block of 32 on every filter tap, so a
// 7x7 filter on 3 channels would multiply 49 x 32 = 1568 deep for 147 values (and C = 3 is
// not addressable by TMA at all: a pixel is 12 bytes).  In NHWC the S*C values a filter row
// needs for one output position are CONTIGUOUS in the input row, so the layer is rewritten
// as a convolution with an R x 1 filter on a packed input
//
//   P[b, h, ow, k] = X[b, h, ow*sw - pad_left + k / C, k % C]   (k < S*C, else 0; 0 outside)
//   V[r, 0, k, f]  = W[r, k / C, k % C, f]                      (k < S*C, else 0)
//   Y = conv(P, V, stride (sh, 1), padding (top, bottom, 0, 0))
//
// with KR = S*C rounded up to 4 channels: K = R * ceil(KR / 32) * 32 (224 for the 7x7x3
// layer).  P costs one pass over B*H*OW*KR floats, written 16 bytes per thread.
__global__ void __launch_bounds__(256)
conv2d_pack_rows_kernel(const float* __restrict__ X, float* __restrict__ P, int rows, int W, int C,
                        int OW, int KR4, int valid, int sw, int pl, const float* __restrict__ Wt,
                        float* __restrict__ V, int filter_total, int F) {
  // the convolution that follows is launched with programmatic stream serialisation: let its
  // CTAs set themselves up while this kernel runs (they wait for its memory before reading)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.y == gridDim.y - 1) {
    // the last row of blocks packs the filter: V[r, k, f] = W[r, k, f] for k < S*C, else 0
    const int KR = KR4 * 4;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < filter_total; i += gridDim.x * blockDim.x) {
      const int f = i % F;
      const int rk = i / F;
      const int k = rk % KR;
      const int r = rk / KR;
      V[i] = k < valid ? __ldg(Wt + (static_cast<int64_t>(r) * valid + k) * F + f) : 0.f;
    }
    return;
  }
  // blockIdx.y walks the B*H input rows four at a time, blockIdx.x * 256 + threadIdx.x the
  // OW * KR4 groups of four packed values of one row: all index arithmetic stays in 32 bits, and
  // a thread has the loads of its four rows in flight before the first store
  const int per_row = OW * KR4;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= per_row) return;
  const int ow = i / KR4;
  const int k0 = (i - ow * KR4) * 4;
  const int row_len = W * C;
  const int e0 = (ow * sw - pl) * C + k0;  // element k of the packed pixel is element e0 + k of the row
  bool ok[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) ok[j] = k0 + j < valid && e0 + j >= 0 && e0 + j < row_len;
  constexpr int ROWS = 4;
  for (int row0 = blockIdx.y * ROWS; row0 < rows; row0 += (gridDim.y - 1) * ROWS) {
    float v[ROWS][4];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float* xr = X + static_cast<int64_t>(row0 + r) * row_len + e0;
#pragma unroll
      for (int j = 0; j < 4; ++j) v[r][j] = (ok[j] && row0 + r < rows) ? __ldg(xr + j) : 0.f;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
      if (row0 + r < rows)
        reinterpret_cast<float4*>(P)[static_cast<int64_t>(row0 + r) * per_row + i] =
            make_float4(v[r][0], v[r][1], v[r][2], v[r][3]);
  }
}

namespace {

int make_tmap_im2col(CUtensorMap* map, const ConvArgs& a, uint32_t pixels) {
  encode_im2col_fn enc = get_encode_im2col();
  if (!enc) {
    set_error("cuTensorMapEncodeIm2col is not available from this driver");
    return XTC_CUDA_ERR_RUNTIME;
  }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W),
                        static_cast<cuuint64_t>(a.H), static_cast<cuuint64_t>(a.B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.C) * 4, static_cast<cuuint64_t>(a.W * a.C) * 4,
                           static_cast<cuuint64_t>(a.H * a.W * a.C) * 4};
  // Base pixels (the input pixel under filter tap (0,0)) range over
  // [-pad, extent + pad - (filter - 1)) in each of W and H.
  // With a stride that does not divide the padded extent the last few input
  // columns / rows are never under tap (0,0): the box ends at the last base pixel,
  // so that it holds exactly OW x OH base pixels whatever the stride.
  const int rem_w = static_cast<int>((a.W + a.pl + a.pr - a.S) % a.sw);
  const int rem_h = static_cast<int>((a.H + a.pt + a.pb - a.R) % a.sh);
  int lower[2] = {-a.pl, -a.pt};
  int upper[2] = {a.pr - static_cast<int>(a.S - 1) - rem_w, a.pb - static_cast<int>(a.R - 1) - rem_h};
  cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(a.sw), static_cast<cuuint32_t>(a.sh), 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(a.X), dims, strides,
                   lower, upper, 32, pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeIm2col failed (%d)", static_cast<int>(r));
    return XTC_CUDA_ERR_INVALID;
  }
  return XTC_CUDA_OK;
}

template <int BN, int KSPANS, bool TMA_STORE>
int launch_conv_tc(const ConvArgs& a) {
  using L = SmemLayout<BN, KSPANS, false>;
  constexpr int BK = L::BK;
  const int max_stages = L::max_stages(TMA_STORE);
  int stages = a.stages <= 0 ? max_stages : a.stages;
  if (stages > max_stages) stages = max_stages;
  if (stages < 2) stages = 2;
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));

  const int64_t M = a.B * a.OH * a.OW, N = a.F, K = a.R * a.S * a.C;
  CUtensorMap tmA, tmB, tmZ, tmC;
  memset(&tmZ, 0, sizeof(tmZ));
  memset(&tmC, 0, sizeof(tmC));
  int rc;
  if ((rc = make_tmap_im2col(&tmA, a, BM))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.Wt, K, N, N, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)))
    return rc;
  if (TMA_STORE &&
      (rc = make_tmap_2d(&tmC, a.Y, M, N, N, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)))
    return rc;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = a.Y;
  p.ldc = N;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.tiles_m = static_cast<int>((M + BM - 1) / BM);
  p.tiles_n = static_cast<int>((N + BN - 1) / BN);
  p.conv_cblocks = static_cast<int>((a.C + BK - 1) / BK);
  p.k_blocks = static_cast<int>(a.R * a.S) * p.conv_cblocks;
  p.chunk_kblocks = p.k_blocks;
  const bool in_cluster = a.cluster_k && BN <= 128;
  const int want_split = in_cluster ? cluster_pieces(p.k_blocks, a.split_k)
                                    : (a.partials && a.counters) ? a.split_k : 1;
  p.split_kblocks = (p.k_blocks + want_split - 1) / want_split;
  p.split_k = (p.k_blocks + p.split_kblocks - 1) / p.split_kblocks;
  p.partials = a.partials;
  p.tile_counters = a.counters;
  if (p.split_k > 1) p.chunk_kblocks = p.split_kblocks;
  p.cluster_k = in_cluster && p.split_k >= 2 && p.split_k <= 8;
  XTC_REQUIRE(p.cluster_k || !in_cluster || p.split_k == 1,
              "conv2d: the cluster split needs 2 to 8 pieces, got %d", p.split_k);
  p.relu = a.relu;
  p.relu_threshold = a.thr;
  p.status = device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "conv2d: device status word unavailable");
  p.conv_ohow = static_cast<int>(a.OH * a.OW);
  p.conv_ow = static_cast<int>(a.OW);
  p.conv_c = static_cast<int>(a.C);
  p.conv_s = static_cast<int>(a.S);
  p.conv_stride_h = a.sh;
  p.conv_stride_w = a.sw;
  p.conv_pad_top = a.pt;
  p.conv_pad_left = a.pl;

  auto kernel = gemm_tf32_kernel<BN, KSPANS, A_IM2COL, true, false, TMA_STORE>;
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
                                             smem, a.stream, tmA, tmB, tmZ, tmZ, tmC, p, stages));
  return XTC_CUDA_OK;
}

// ---- resident weights + halo tiles (conv2d_halo.cuh) ------------------------------
struct HaloPlan {
  bool ok = false;
  int bn = 0, stages = 0, P = 0, stage_bytes = 0, nslab = 0, nblk = 0, slab = 32, smem = 0;
};

// Whether the halo kernel can run this convolution, and with what footprint.
// pair = the CTA-pair kernel, where each CTA keeps half of the filter columns.
// slab = channels per pipeline stage (32, or 16 in the single-CTA kernel).
// taps = the two-taps-per-MMA kernel (conv2d_halo_taps.cuh): at most 64 filters, a filter
// row of at least two taps, one CTA per tile, 1 KB more for the rows that cross warps.
HaloPlan plan_halo(const ConvArgs& a, bool pair = false, int slab = 32, bool taps = false) {
  HaloPlan h;
  h.slab = slab;
  if (a.sh != 1 || a.sw != 1 || a.F > 256) return h;
  if (taps && (pair || a.F > 64 || a.S < 2)) return h;
  const int64_t Wp = a.W + a.pl + a.pr;
  const int64_t P = BM + (a.R - 1) * Wp + (a.S - 1);
  if (P > 1024 || a.pl > 127 || a.pt > 127 || a.pr > 127 || a.pb > 127) return h;
  h.bn = a.F <= 64 ? 64 : (a.F <= 128 ? 128 : 256);
  h.P = static_cast<int>(P);
  h.stage_bytes = static_cast<int>((P * slab * 4 + 1023) / 1024 * 1024);
  h.nslab = static_cast<int>((a.C + slab - 1) / slab);
  h.nblk = static_cast<int>((a.C + 31) / 32);
  const int64_t wbytes = a.R * a.S * h.nblk * (pair ? h.bn / 2 : h.bn) * 128;
  const int64_t fixed = 1024 + 1024 + (taps ? 1024 : 0);  // alignment slack, barriers, exchange rows
  const int64_t budget = 232448 - fixed;
  const int64_t stages = (budget - wbytes) / h.stage_bytes;
  if (stages < 2) return h;
  h.stages = static_cast<int>(stages > 8 ? 8 : stages);
  h.smem = static_cast<int>(fixed + wbytes + static_cast<int64_t>(h.stages) * h.stage_bytes);
  h.ok = true;
  return h;
}

template <int BN, bool PAIR, int SLAB, bool TAPS = false>
int launch_conv_halo(const ConvArgs& a, const HaloPlan& h) {
  encode_im2col_fn enc = get_encode_im2col();
  XTC_REQUIRE(enc != nullptr, "cuTensorMapEncodeIm2col is not available from this driver");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  const int64_t Hp = a.H + a.pt + a.pb, Wp = a.W + a.pl + a.pr;
  // One copy = P consecutive pixels of the zero-padded image grid: the bounding
  // box is the padded image, so the traversal wraps rows and images by itself.
  CUtensorMap tmX, tmW;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W),
                        static_cast<cuuint64_t>(a.H), static_cast<cuuint64_t>(a.B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.C) * 4, static_cast<cuuint64_t>(a.W * a.C) * 4,
                           static_cast<cuuint64_t>(a.H * a.W * a.C) * 4};
  int lower[2] = {-a.pl, -a.pt};
  int upper[2] = {a.pr, a.pb};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(a.X), dims, strides,
                   lower, upper, SLAB, static_cast<cuuint32_t>(h.P), estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   SLAB == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  XTC_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeIm2col (halo) failed (%d)", static_cast<int>(r));
  int rc;
  if ((rc = make_tmap_2d(&tmW, a.Wt, a.R * a.S * a.C, a.F, a.F, 32, 32,
                         CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)))
    return rc;

  ConvHaloParams p;
  memset(&p, 0, sizeof(p));
  p.Y = a.Y;
  p.status = device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "conv2d: device status word unavailable");
  p.Q = a.B * Hp * Wp;
  const int tile_positions = TAPS ? TAPS_TILE : PAIR ? 2 * BM : BM;
  p.tiles = static_cast<int>((p.Q + tile_positions - 1) / tile_positions);
  p.Hp = static_cast<int>(Hp);
  p.Wp = static_cast<int>(Wp);
  p.OH = static_cast<int>(a.OH);
  p.OW = static_cast<int>(a.OW);
  p.F = static_cast<int>(a.F);
  p.nslab = h.nslab;
  p.nblk = h.nblk;
  p.C = static_cast<int>(a.C);
  p.taps = static_cast<int>(a.R * a.S);
  p.S = static_cast<int>(a.S);
  p.pad_left = a.pl;
  p.pad_top = a.pt;
  p.stage_bytes = h.stage_bytes;
  p.stage_tx = h.P * SLAB * 4;
  p.stages = a.stages >= 2 && a.stages < h.stages ? a.stages : h.stages;
  p.relu = a.relu;
  p.relu_threshold = a.thr;

  // two issuing threads whenever both accumulators fit in TMEM and there are taps to share
  constexpr bool CAN_DUAL = BN <= 128;
  const bool dual = CAN_DUAL && p.taps >= 2;
  static_assert(!PAIR || SLAB == 32, "the CTA-pair kernel has 32-channel slabs only");
  static_assert(!TAPS || (BN == 64 && !PAIR), "two taps per MMA: 64 filters, one CTA per tile");
  auto kernel = TAPS ? conv2d_halo_taps_kernel<SLAB>
                : PAIR ? (dual ? conv2d_halo_pair_kernel<BN, CAN_DUAL> : conv2d_halo_pair_kernel<BN, false>)
                       : (dual ? conv2d_halo_kernel<BN, CAN_DUAL, SLAB>
                               : conv2d_halo_kernel<BN, false, SLAB>);
  static thread_local int configured_dev[2] = {-1, -1};
  static thread_local int configured_smem[2] = {0, 0};
  const int which = dual ? 1 : 0;
  if (configured_dev[which] != dev || configured_smem[which] < h.smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem));
    configured_dev[which] = dev;
    configured_smem[which] = h.smem;
  }
  const int slots = PAIR ? sm_count(dev) / 2 : sm_count(dev);
  const int grid = (p.tiles < slots ? p.tiles : slots) * (PAIR ? 2 : 1);
  XTC_CUDA_CHECK(launch_overlapped(kernel, grid, HALO_THREADS, h.smem, a.stream, tmX, tmW, p));
  return XTC_CUDA_OK;
}

template <int BN>
int dispatch_conv_halo_bn(const ConvArgs& a, const HaloPlan& h, bool pair) {
  if (pair) return launch_conv_halo<BN, true, 32>(a, h);
  return h.slab == 16 ? launch_conv_halo<BN, false, 16>(a, h) : launch_conv_halo<BN, false, 32>(a, h);
}

// The sliding-window form of the resident-weights kernel (conv2d_halo_slide.cuh): stride 1,
// at most 128 filters, a halo run of at most 256 positions, the filter bank beside five
// 16 KB ring slots.
struct SlidePlan {
  bool ok = false;
  int bn = 0, nslab = 0, nblk = 0, smem = 0;
};
SlidePlan plan_slide(const ConvArgs& a) {
  SlidePlan s;
  if (a.sh != 1 || a.sw != 1 || a.F > 128 || a.R * a.S < 2) return s;  // two threads share the taps
  const int64_t Wp = a.W + a.pl + a.pr;
  const int64_t P = BM + (a.R - 1) * Wp + (a.S - 1);
  if (P > 2 * SLIDE_CHUNK || a.pl > 127 || a.pt > 127 || a.pr > 127 || a.pb > 127) return s;
  s.bn = a.F <= 64 ? 64 : 128;
  s.nblk = static_cast<int>((a.C + 31) / 32);
  s.nslab = s.nblk;
  const int64_t wbytes = a.R * a.S * s.nblk * s.bn * 128;
  const int64_t total = 1024 + wbytes + (SLIDE_SLOTS + 1) * SLIDE_SLOT_BYTES + 1024;
  if (total > 232448) return s;
  s.smem = static_cast<int>(total);
  s.ok = true;
  return s;
}

template <int BN>
int launch_conv_slide(const ConvArgs& a, const SlidePlan& h) {
  encode_im2col_fn enc = get_encode_im2col();
  XTC_REQUIRE(enc != nullptr, "cuTensorMapEncodeIm2col is not available from this driver");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  const int64_t Hp = a.H + a.pt + a.pb, Wp = a.W + a.pl + a.pr;
  CUtensorMap tmX, tmW;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W),
                        static_cast<cuuint64_t>(a.H), static_cast<cuuint64_t>(a.B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.C) * 4, static_cast<cuuint64_t>(a.W * a.C) * 4,
                           static_cast<cuuint64_t>(a.H * a.W * a.C) * 4};
  int lower[2] = {-a.pl, -a.pt};
  int upper[2] = {a.pr, a.pb};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  // one copy = 128 consecutive positions of the zero-padded image grid, 32 channels
  CUresult r = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(a.X), dims, strides,
                   lower, upper, 32, SLIDE_CHUNK, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  XTC_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeIm2col (sliding halo) failed (%d)", static_cast<int>(r));
  int rc;
  if ((rc = make_tmap_2d(&tmW, a.Wt, a.R * a.S * a.C, a.F, a.F, 32, 32,
                         CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)))
    return rc;
  ConvHaloParams p;
  memset(&p, 0, sizeof(p));
  p.Y = a.Y;
  p.status = device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "conv2d: device status word unavailable");
  p.Q = a.B * Hp * Wp;
  p.tiles = static_cast<int>((p.Q + BM - 1) / BM);
  p.Hp = static_cast<int>(Hp);
  p.Wp = static_cast<int>(Wp);
  p.OH = static_cast<int>(a.OH);
  p.OW = static_cast<int>(a.OW);
  p.F = static_cast<int>(a.F);
  p.nslab = h.nslab;
  p.nblk = h.nblk;
  p.C = static_cast<int>(a.C);
  p.taps = static_cast<int>(a.R * a.S);
  p.S = static_cast<int>(a.S);
  p.pad_left = a.pl;
  p.pad_top = a.pt;
  p.relu = a.relu;
  p.relu_threshold = a.thr;
  auto kernel = conv2d_halo_slide_kernel<BN>;
  static thread_local int configured_dev = -1;
  static thread_local int configured_smem = 0;
  if (configured_dev != dev || configured_smem < h.smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem));
    configured_dev = dev;
    configured_smem = h.smem;
  }
  const int slots = sm_count(dev);
  const int grid = p.tiles < slots ? p.tiles : slots;
  XTC_CUDA_CHECK(launch_overlapped(kernel, grid, SLIDE_THREADS, h.smem, a.stream, tmX, tmW, p));
  return XTC_CUDA_OK;
}

// The streamed-weights form (conv2d_halo_stream.cuh): stride 1, CTA pairs, a stage = one
// 32-channel halo slab + the weights of every tap for this CTA's 64 filters; at least two stages.
struct StreamPlan {
  bool ok = false;
  int P = 0, stages = 0, stage_bytes = 0, wts_offset = 0, wts_tx = 0, nslab = 0, smem = 0, slab = 32;
};
StreamPlan plan_stream(const ConvArgs& a, int slab = 32) {
  StreamPlan s;
  s.slab = slab;
  if (a.sh != 1 || a.sw != 1 || a.C % 4 != 0 || a.F % 4 != 0) return s;
  const int64_t taps = a.R * a.S;
  if (taps < 2 || taps > 32) return s;  // a single tap is a plain GEMM: nothing to share
  const int64_t Wp = a.W + a.pl + a.pr;
  const int64_t P = BM + (a.R - 1) * Wp + (a.S - 1);
  if (P > 1024 || a.pl > 127 || a.pt > 127 || a.pr > 127 || a.pb > 127) return s;
  s.P = static_cast<int>(P);
  s.wts_offset = static_cast<int>((P * slab * 4 + 1023) / 1024 * 1024);
  s.wts_tx = static_cast<int>(taps * (STREAM_BN / 2) * slab * 4);
  s.stage_bytes = s.wts_offset + s.wts_tx;
  const int64_t fixed = 1024 + 1024;  // alignment slack, barriers
  const int64_t stages = (232448 - fixed) / s.stage_bytes;
  if (stages < 2) return s;
  s.stages = static_cast<int>(stages > 6 ? 6 : stages);
  s.nslab = static_cast<int>((a.C + slab - 1) / slab);
  s.smem = static_cast<int>(fixed + static_cast<int64_t>(s.stages) * s.stage_bytes);
  s.ok = true;
  return s;
}

// Workspace of the balanced form of the streamed-weights kernel (see conv2d_halo_stream.cuh):
// one flag and one 32 x 128 block of partial sums per (CTA pair, CTA, epilogue warp).
static size_t stream_flag_bytes(int pairs) { return (static_cast<size_t>(pairs) * 8 * 4 + 255) & ~static_cast<size_t>(255); }
static size_t stream_balance_bytes(int pairs) {
  return stream_flag_bytes(pairs) + static_cast<size_t>(pairs) * 8 * 32 * STREAM_BN * 4;
}
// Whether dealing out (work item, slab) units evenly beats whole items round-robin.  A pair
// then has up to two partial items, each with an epilogue of its own and a pass over the
// partial sums, about two slabs' worth of time, so the longest pair's units must shrink by more
// than that (us, balanced / round-robin: 16x28x28x256 -> 512, 25 units against 32, 44.8 / 47.8;
// but 32x28x28x128 -> 128, 7 against 8, 19.9 / 17.3 and 32x14x14x256 -> 256, 7 against 8,
// 20.9 / 16.8).  And every pair must hold two items' worth of units, so that an item is cut
// once at most: cut into many pieces, the pair that stores an item waits for all the others
// and sums their partials alone (8x14x14x256 -> 256, 2 units against 8: 20.4 / 16.0).
static bool stream_balance_pays(int64_t items, int nslab, int pairs) {
  const int64_t units = items * nslab;
  if (units < 2ll * nslab * pairs) return false;
  const int64_t plain = (items + pairs - 1) / pairs * nslab;
  const int64_t even = (units + pairs - 1) / pairs;
  return (even + 2) * 100 <= plain * 85;
}

// Nothing named and no room for the whole filter bank beside one CTA's stages: stream the
// weights with the halo slabs (conv2d_halo_stream.cuh) where there is work for most CTA pairs
// (or at most two channel slabs to walk) and most positions of the padded grid are outputs.
// Measured against the im2col kernels (us, batch 32): 28x28x128 -> 128 17.3 / 23.6, 14x14x256 ->
// 256 16.8 / 21.4, 56x56x64 -> 128 26.9 / 36.5 (half a bank per CTA of a pair), 28x28x128 -> 256
// 27.3 / 31.0; 27x27x48 -> 192 (8 work items, two slabs) 8.2 / 10.3; but 7x7x512 -> 512 27.7 /
// 26.0 (49 of 81 positions are outputs) and 8x14x14x256 -> 256 16.0 / 12.1 (16 work items).
static bool stream_is_default(const ConvArgs& a, const StreamPlan& sp) {
  if (!sp.ok) return false;
  const int64_t grid_positions = (a.H + a.pt + a.pb) * (a.W + a.pl + a.pr);
  const int64_t items = (a.B * grid_positions + 2 * BM - 1) / (2 * BM) * ((a.F + STREAM_BN - 1) / STREAM_BN);
  return (items >= 40 || sp.nslab <= 2) && a.OH * a.OW * 10 >= grid_positions * 7;
}

template <int SLAB>
int launch_conv_stream_slab(const ConvArgs& a, const StreamPlan& h, void* workspace, size_t workspace_bytes) {
  encode_im2col_fn enc = get_encode_im2col();
  encode_tiled_fn enc_tiled = get_encode_tiled();
  XTC_REQUIRE(enc != nullptr && enc_tiled != nullptr,
              "cuTensorMapEncodeIm2col / Tiled are not available from this driver");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  const int64_t Hp = a.H + a.pt + a.pb, Wp = a.W + a.pl + a.pr;
  CUtensorMap tmX, tmW;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(a.C), static_cast<cuuint64_t>(a.W),
                        static_cast<cuuint64_t>(a.H), static_cast<cuuint64_t>(a.B)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(a.C) * 4, static_cast<cuuint64_t>(a.W * a.C) * 4,
                           static_cast<cuuint64_t>(a.H * a.W * a.C) * 4};
  int lower[2] = {-a.pl, -a.pt};
  int upper[2] = {a.pr, a.pb};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(a.X), dims, strides,
                   lower, upper, SLAB, static_cast<cuuint32_t>(h.P), estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   SLAB == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  XTC_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeIm2col (streamed halo) failed (%d)", static_cast<int>(r));
  // the filter as [tap][channel][filter]: one copy = every tap x 32 channels x 32 filters
  const int taps = static_cast<int>(a.R * a.S);
  cuuint64_t wdims[3] = {static_cast<cuuint64_t>(a.F), static_cast<cuuint64_t>(a.C),
                         static_cast<cuuint64_t>(taps)};
  cuuint64_t wstrides[2] = {static_cast<cuuint64_t>(a.F) * 4, static_cast<cuuint64_t>(a.C * a.F) * 4};
  cuuint32_t wbox[3] = {32, SLAB, static_cast<cuuint32_t>(taps)};
  r = enc_tiled(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(a.Wt), wdims, wstrides, wbox,
                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  XTC_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (streamed weights) failed (%d)", static_cast<int>(r));

  ConvHaloParams p;
  memset(&p, 0, sizeof(p));
  p.Y = a.Y;
  p.status = device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "conv2d: device status word unavailable");
  p.Q = a.B * Hp * Wp;
  p.ntiles_n = static_cast<int>((a.F + STREAM_BN - 1) / STREAM_BN);
  const int64_t tiles = (p.Q + 2 * BM - 1) / (2 * BM) * p.ntiles_n;
  XTC_REQUIRE(tiles < (1ll << 31), "conv2d: %lld work items", static_cast<long long>(tiles));
  p.tiles = static_cast<int>(tiles);
  p.Hp = static_cast<int>(Hp);
  p.Wp = static_cast<int>(Wp);
  p.OH = static_cast<int>(a.OH);
  p.OW = static_cast<int>(a.OW);
  p.F = static_cast<int>(a.F);
  p.nslab = h.nslab;
  p.nblk = h.nslab;
  p.C = static_cast<int>(a.C);
  p.taps = taps;
  p.S = static_cast<int>(a.S);
  p.pad_left = a.pl;
  p.pad_top = a.pt;
  p.stage_bytes = h.stage_bytes;
  p.stage_tx = h.P * SLAB * 4;
  p.wts_offset = h.wts_offset;
  p.wts_tx = h.wts_tx;
  p.stages = a.stages >= 2 && a.stages < h.stages ? a.stages : h.stages;
  p.relu = a.relu;
  p.relu_threshold = a.thr;
  auto kernel = conv2d_halo_stream_kernel<true, SLAB>;  // plan_stream wants two taps or more
  static thread_local int configured_dev = -1;
  static thread_local int configured_smem = 0;
  if (configured_dev != dev || configured_smem < h.smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem));
    configured_dev = dev;
    configured_smem = h.smem;
  }
  const int slots = sm_count(dev) / 2;
  int grid = (p.tiles < slots ? p.tiles : slots) * 2;
  if (workspace != nullptr && workspace_bytes >= stream_balance_bytes(slots) &&
      (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 && stream_balance_pays(p.tiles, p.nslab, slots)) {
    // every pair of the device, each with an even share of the (item, slab) units; the flags
    // at the start of the workspace are zero (first use) or were left zero by the last launch
    p.sk_flags = static_cast<int*>(workspace);
    p.sk_partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + stream_flag_bytes(slots));
    grid = slots * 2;
  }
  XTC_CUDA_CHECK(launch_overlapped(kernel, grid, HALO_THREADS, h.smem, a.stream, tmX, tmW, p));
  return XTC_CUDA_OK;
}

int launch_conv_stream(const ConvArgs& a, const StreamPlan& h, void* workspace = nullptr,
                       size_t workspace_bytes = 0) {
  return h.slab == 16 ? launch_conv_stream_slab<16>(a, h, workspace, workspace_bytes)
                      : launch_conv_stream_slab<32>(a, h, workspace, workspace_bytes);
}

int dispatch_conv_halo(const ConvArgs& a, const HaloPlan& h, bool pair, bool taps = false) {
  if (taps)
    return h.slab == 16 ? launch_conv_halo<64, false, 16, true>(a, h)
                        : launch_conv_halo<64, false, 32, true>(a, h);
  switch (h.bn) {
    case 64: return dispatch_conv_halo_bn<64>(a, h, pair);
    case 128: return dispatch_conv_halo_bn<128>(a, h, pair);
    default: return dispatch_conv_halo_bn<256>(a, h, pair);
  }
}

// 256 output pixels per CTA pair: each CTA fetches its own 128 pixels and half of
// the filter columns.
template <int BN, int KSPANS>
int launch_conv_pair(const ConvArgs& a) {
  using L = PairSmem<BN, KSPANS>;
  constexpr int BK = L::BK;
  const int max_stages = L::max_stages();
  int stages = a.stages <= 0 ? max_stages : a.stages;
  if (stages > max_stages) stages = max_stages;
  if (stages < 2) stages = 2;
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  const int64_t M = a.B * a.OH * a.OW, N = a.F, K = a.R * a.S * a.C;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_tmap_im2col(&tmA, a, BM))) return rc;
  if ((rc = make_tmap_2d(&tmB, a.Wt, K, N, N, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))) return rc;
  if ((rc = make_tmap_2d(&tmC, a.Y, M, N, N, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.C = a.Y;
  p.ldc = N;
  p.M = static_cast<int>(M);
  p.N = static_cast<int>(N);
  p.K = static_cast<int>(K);
  p.tiles_m = static_cast<int>((M + 2 * BM - 1) / (2 * BM));
  p.tiles_n = static_cast<int>((N + BN - 1) / BN);
  p.conv_cblocks = static_cast<int>((a.C + BK - 1) / BK);
  p.k_blocks = static_cast<int>(a.R * a.S) * p.conv_cblocks;
  p.chunk_kblocks = p.k_blocks;
  p.relu = a.relu;
  p.relu_threshold = a.thr;
  p.status = device_status_word(dev);
  XTC_REQUIRE(p.status != nullptr, "conv2d: device status word unavailable");
  p.conv_ohow = static_cast<int>(a.OH * a.OW);
  p.conv_ow = static_cast<int>(a.OW);
  p.conv_c = static_cast<int>(a.C);
  p.conv_s = static_cast<int>(a.S);
  p.conv_stride_h = a.sh;
  p.conv_stride_w = a.sw;
  p.conv_pad_top = a.pt;
  p.conv_pad_left = a.pl;
  auto kernel = gemm_tf32_pair_kernel<BN, KSPANS, A_IM2COL, true>;
  const int smem = L::total(stages);
  static thread_local int configured_dev = -1;
  static thread_local int configured_smem = 0;
  if (configured_dev != dev || configured_smem < smem) {
    XTC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured_dev = dev;
    configured_smem = smem;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int max_pairs = sm_count(dev) / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  p.group_n = panel_columns(pairs, 2 * BM, BN, p.tiles_n);
  XTC_CUDA_CHECK(launch_overlapped(kernel, 2 * pairs, NUM_THREADS, smem, a.stream, tmA, tmB, tmC, p,
                                   stages));
  return XTC_CUDA_OK;
}

int dispatch_conv_pair(const ConvArgs& a, int tile_n, int tile_k) {
  const int ks = tile_k == 64 ? 2 : 1;
  switch (tile_n) {
    case 64: return ks == 1 ? launch_conv_pair<64, 1>(a) : launch_conv_pair<64, 2>(a);
    case 128: return ks == 1 ? launch_conv_pair<128, 1>(a) : launch_conv_pair<128, 2>(a);
    case 256: return ks == 1 ? launch_conv_pair<256, 1>(a) : launch_conv_pair<256, 2>(a);
  }
  set_error("conv2d: unsupported tile_n=%d", tile_n);
  return XTC_CUDA_ERR_UNSUPPORTED;
}

template <bool TMA_STORE>
int dispatch_conv(const ConvArgs& a, int tile_n, int tile_k) {
  const int ks = tile_k == 64 ? 2 : 1;
  switch (tile_n) {
    case 64: return ks == 1 ? launch_conv_tc<64, 1, TMA_STORE>(a) : launch_conv_tc<64, 2, TMA_STORE>(a);
    case 128: return ks == 1 ? launch_conv_tc<128, 1, TMA_STORE>(a) : launch_conv_tc<128, 2, TMA_STORE>(a);
    case 256: return ks == 1 ? launch_conv_tc<256, 1, TMA_STORE>(a) : launch_conv_tc<256, 2, TMA_STORE>(a);
  }
  set_error("conv2d: unsupported tile_n=%d", tile_n);
  return XTC_CUDA_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace xtc

using namespace xtc;

// Split-K workspace of the im2col kernel for a layer whose caller named nothing:
// tile counters, then split x tiles partial tiles of 128 x tile_n floats.
static size_t conv_split_bytes(int64_t M, int64_t F, const AutoChoice& pick) {
  if (pick.tile_m != BM || pick.split_k <= 1) return 0;
  const size_t tiles = static_cast<size_t>((M + BM - 1) / BM) * ((F + pick.tile_n - 1) / pick.tile_n);
  return ((tiles * 4 + 255) & ~static_cast<size_t>(255)) +
         static_cast<size_t>(pick.split_k) * tiles * BM * pick.tile_n * 4;
}
// A split the im2col launcher reduces inside a thread-block cluster (no workspace): 2 to 8
// pieces of a tile at most 128 filters wide, with every cluster resident at once.
static bool conv_split_in_cluster(int64_t M, int64_t F, const AutoChoice& pick, int dev) {
  if (pick.tile_m != BM || pick.tile_n > 128 || F % 4 != 0) return false;
  if (pick.split_k < 2 || pick.split_k > 8) return false;
  const int64_t tiles = ((M + BM - 1) / BM) * ((F + pick.tile_n - 1) / pick.tile_n);
  return tiles <= cluster_capacity(dev, pick.split_k);
}
static bool conv_names_nothing(const xtc_cuda_gemm_config& c) {
  return c.precision == XTC_CUDA_PRECISION_TF32 && c.variant == 0 && c.tile_m == 0 && c.tile_n == 0 &&
         c.tile_k == 0 && c.split_k == 0;
}

// The packed form of a thin-input layer (see conv2d_pack_rows_kernel): whether it applies and
// how much workspace the packed input and filter take (each rounded up to 256 bytes).
struct ThinPlan {
  bool ok = false;
  int64_t KR = 0, OW = 0;
  size_t p_bytes = 0, v_bytes = 0;
};
static ThinPlan plan_thin(int64_t B, int64_t H, int64_t W, int64_t C, int64_t R, int64_t S, int64_t F,
                          int sh, int sw, int pt, int pb, int pl, int pr,
                          const xtc_cuda_gemm_config& c) {
  ThinPlan t;
  // layers the tensor-core kernels cannot address (C not a multiple of 4), and aligned ones of
  // at most 8 channels when the caller named no kernel parameter
  bool thin = C % 4 != 0;
  if (!thin && C <= 8 && S > 1) {
    // aligned and thin: the resident-weights kernel is the faster where it applies (stride 1;
    // 32x58x58x8 -> 64, 3x3: 12.6 us against 22.6 us packed), the packed form elsewhere
    // (453x453x8 -> 64, 7x7 stride 2: 33.3 us against 57.6 us)
    ConvArgs a;
    memset(&a, 0, sizeof(a));
    a.B = B; a.H = H; a.W = W; a.C = C; a.R = R; a.S = S; a.F = F;
    a.sh = sh; a.sw = sw; a.pt = pt; a.pb = pb; a.pl = pl; a.pr = pr;
    thin = !(plan_halo(a, false, 32).ok || plan_halo(a, false, 16).ok || plan_halo(a, true, 32).ok);
  }
  if (B * H > 0x7fffffff || W * C > 0x3fffffff || R * ((S * C + 3) / 4 * 4) * F > 0x7fffffff) return t;
  if (!thin || c.precision != XTC_CUDA_PRECISION_TF32 || F % 4 != 0 || S * C > 1024 || R > 120 ||
      !(c.variant == 0 && c.tile_m == 0 && c.tile_n == 0 && c.tile_k == 0 && c.split_k == 0))
    return t;
  t.OW = (W + pl + pr - S) / sw + 1;
  if (t.OW <= 0 || t.OW > 65535 || H > 65535) return t;
  t.KR = (S * C + 3) / 4 * 4;
  const size_t round = 255;
  t.p_bytes = (static_cast<size_t>(B * H * t.OW * t.KR) * 4 + round) & ~round;
  t.v_bytes = (static_cast<size_t>(R * t.KR * F) * 4 + round) & ~round;
  t.ok = true;
  return t;
}

extern "C" int xtc_cuda_conv2d_workspace_bytes(int64_t B, int64_t H, int64_t W, int64_t C, int64_t R,
                                               int64_t S, int64_t F, int stride_h, int stride_w,
                                               int pad_top, int pad_bottom, int pad_left,
                                               int pad_right, const xtc_cuda_gemm_config* cfg,
                                               size_t* bytes) {
  XTC_REQUIRE(bytes != nullptr, "conv2d_workspace_bytes: bytes is NULL");
  *bytes = 0;
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || R <= 0 || S <= 0 || F <= 0 || stride_h <= 0 ||
      stride_w <= 0 || H + pad_top + pad_bottom < R || W + pad_left + pad_right < S)
    return XTC_CUDA_OK;  // the convolution itself reports what is wrong
  xtc_cuda_gemm_config c;
  memset(&c, 0, sizeof(c));
  if (cfg) c = *cfg;
  const int64_t OH = (H + pad_top + pad_bottom - R) / stride_h + 1;
  const int64_t OW = (W + pad_left + pad_right - S) / stride_w + 1;
  const int64_t M = B * OH * OW;
  if (R == 1 && S == 1 && stride_h == 1 && stride_w == 1 &&
      pad_top + pad_bottom + pad_left + pad_right == 0 && c.variant == 0 &&
      c.precision != XTC_CUDA_PRECISION_3XTF32)
    return xtc_cuda_gemm_workspace_bytes(M, F, C, 0, &c, bytes);
  if (const ThinPlan t = plan_thin(B, H, W, C, R, S, F, stride_h, stride_w, pad_top, pad_bottom, pad_left, pad_right, c); t.ok) {
    size_t inner = 0;
    const int rc = xtc_cuda_conv2d_workspace_bytes(B, H, t.OW, t.KR, R, 1, F, stride_h, 1, pad_top,
                                                   pad_bottom, 0, 0, nullptr, &inner);
    if (rc != XTC_CUDA_OK) return rc;
    *bytes = t.p_bytes + t.v_bytes + inner;
    return XTC_CUDA_OK;
  }
  ConvArgs a;
  memset(&a, 0, sizeof(a));
  a.B = B; a.H = H; a.W = W; a.C = C; a.R = R; a.S = S; a.F = F;
  a.sh = stride_h; a.sw = stride_w;
  a.pt = pad_top; a.pb = pad_bottom; a.pl = pad_left; a.pr = pad_right;
  a.OH = OH; a.OW = OW;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) sms = sm_count(dev); else cudaGetLastError();
  // streamed weights (asked for, or the library's own choice): flags and partial sums of the
  // balanced form, where dealing out (item, slab) units evenly shortens the longest pair
  auto stream_bytes = [&](const StreamPlan& sp) -> size_t {
    const int64_t items = (B * (H + pad_top + pad_bottom) * (W + pad_left + pad_right) + 2 * BM - 1) /
                          (2 * BM) * ((F + STREAM_BN - 1) / STREAM_BN);
    return stream_balance_pays(items, sp.nslab, sms / 2) ? stream_balance_bytes(sms / 2) : 0;
  };
  if (c.variant == 5) {
    const StreamPlan sp = plan_stream(a);
    if (sp.ok) *bytes = stream_bytes(sp);
    return XTC_CUDA_OK;
  }
  if (!conv_names_nothing(c)) return XTC_CUDA_OK;
  if (plan_halo(a, false, 32).ok || plan_halo(a, false, 16).ok)
    return XTC_CUDA_OK;  // resident weights in one CTA: no workspace
  if (const StreamPlan sp = plan_stream(a); stream_is_default(a, sp)) {
    *bytes = stream_bytes(sp);
    return XTC_CUDA_OK;
  }
  if (plan_halo(a, true, 32).ok || plan_halo(a, false, 32, true).ok || plan_halo(a, false, 16, true).ok)
    return XTC_CUDA_OK;  // resident weights: no workspace
  int caps[9] = {};
  for (int sz = 2; sz <= 8; ++sz) caps[sz] = cluster_capacity(dev, sz);
  const AutoChoice pick =
      choose_tf32_default(M, F, R * S * ((C + 31) / 32 * 32), sms, true, true, F % 4 == 0 ? caps : nullptr,
                          false);
  *bytes = conv_split_in_cluster(M, F, pick, dev) ? 0 : conv_split_bytes(M, F, pick);
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_conv2d_nhwc_f32(const float* X, const float* Wt, float* Y, int64_t B,
                                        int64_t H, int64_t W, int64_t C, int64_t R, int64_t S,
                                        int64_t F, int stride_h, int stride_w, int pad_top,
                                        int pad_bottom, int pad_left, int pad_right, int flags,
                                        float relu_threshold, const xtc_cuda_gemm_config* cfg,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  XTC_REQUIRE(X && Wt && Y, "conv2d: NULL operand");
  XTC_REQUIRE(B > 0 && H > 0 && W > 0 && C > 0 && R > 0 && S > 0 && F > 0, "conv2d: empty extent");
  XTC_REQUIRE(stride_h > 0 && stride_w > 0, "conv2d: stride must be positive");
  XTC_REQUIRE(pad_top >= 0 && pad_bottom >= 0 && pad_left >= 0 && pad_right >= 0,
              "conv2d: negative padding");
  ConvArgs a;
  a.X = X; a.Wt = Wt; a.Y = Y;
  a.B = B; a.H = H; a.W = W; a.C = C; a.R = R; a.S = S; a.F = F;
  a.sh = stride_h; a.sw = stride_w;
  a.pt = pad_top; a.pb = pad_bottom; a.pl = pad_left; a.pr = pad_right;
  XTC_REQUIRE(H + pad_top + pad_bottom >= R && W + pad_left + pad_right >= S,
              "conv2d: filter larger than the padded input");
  a.OH = (H + pad_top + pad_bottom - R) / stride_h + 1;
  a.OW = (W + pad_left + pad_right - S) / stride_w + 1;
  a.relu = flags & XTC_CUDA_FUSE_RELU;
  a.thr = relu_threshold;
  xtc_cuda_gemm_config c;
  memset(&c, 0, sizeof(c));
  if (cfg) c = *cfg;
  a.stages = c.stages;
  a.stream = static_cast<cudaStream_t>(stream);
  const int64_t M = B * a.OH * a.OW;
  XTC_REQUIRE(M < (1ll << 31) && R * S * C < (1ll << 31), "conv2d: problem too large");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));

  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  // A 1x1 filter with unit stride and no padding is a plain matrix product
  // [B*H*W, C] x [C, F]: the GEMM entry point picks kernel and tile for it.
  if (R == 1 && S == 1 && stride_h == 1 && stride_w == 1 && pad_top + pad_bottom + pad_left + pad_right == 0 &&
      c.variant == 0 && c.precision != XTC_CUDA_PRECISION_3XTF32)
    return xtc_cuda_gemm_f32(X, Wt, Y, M, F, C, C, F, F, flags & XTC_CUDA_FUSE_RELU, relu_threshold,
                             &c, workspace, workspace_bytes, stream);
  // The tensor-core path needs TMA-addressable operands, a unit or small
  // traversal stride, and corner offsets within the im2col descriptor's range.
  // Thin inputs: pack filter rows and run the R x 1 layer on the tensor cores, when the caller
  // brought the workspace for it (xtc_cuda_conv2d_workspace_bytes); without, the layer runs as
  // it did (the CUDA-core kernel when C is not a multiple of 4).
  if (const ThinPlan t = plan_thin(B, H, W, C, R, S, F, stride_h, stride_w, pad_top, pad_bottom, pad_left, pad_right, c);
      t.ok && workspace != nullptr && workspace_bytes >= t.p_bytes + t.v_bytes &&
      (reinterpret_cast<uintptr_t>(workspace) & 15) == 0 && a16(Y)) {
    float* P = static_cast<float*>(workspace);
    float* V = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + t.p_bytes);
    const int64_t rows = B * H;
    const int per_row = static_cast<int>(t.OW * (t.KR / 4));
    // one launch: a row of blocks per four input rows packs the input, one more packs the filter
    const int64_t row_groups = (rows + 3) / 4;
    const dim3 pack_grid(static_cast<unsigned>((per_row + 255) / 256),
                         static_cast<unsigned>((row_groups < 65534 ? row_groups : 65534) + 1));
    conv2d_pack_rows_kernel<<<pack_grid, 256, 0, a.stream>>>(
        X, P, static_cast<int>(rows), static_cast<int>(W), static_cast<int>(C), static_cast<int>(t.OW),
        static_cast<int>(t.KR / 4), static_cast<int>(S * C), stride_w, pad_left, Wt, V,
        static_cast<int>(R * t.KR * F), static_cast<int>(F));
    XTC_CUDA_CHECK(cudaGetLastError());
    uint8_t* rest = static_cast<uint8_t*>(workspace) + t.p_bytes + t.v_bytes;
    return xtc_cuda_conv2d_nhwc_f32(P, V, Y, B, H, t.OW, t.KR, R, 1, F, stride_h, 1, pad_top, pad_bottom,
                                    0, 0, flags, relu_threshold, nullptr, rest,
                                    workspace_bytes - t.p_bytes - t.v_bytes, stream);
  }
  const bool tc_ok = c.precision == XTC_CUDA_PRECISION_TF32 && C % 4 == 0 && F % 4 == 0 &&
                     a16(X) && a16(Wt) && stride_h <= 8 && stride_w <= 8 && pad_top <= 127 &&
                     pad_left <= 127 && pad_right <= 127 && pad_bottom <= 127 && S <= 120 &&
                     R <= 120 && W <= 65535 && H <= 65535;
  if (!tc_ok) {
    XTC_REQUIRE(c.precision != XTC_CUDA_PRECISION_3XTF32,
                "conv2d: the 3xTF32 mode is not available for convolutions");
    const int64_t total = M * F;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count(dev)) * 16;
    if (blocks > cap) blocks = cap;
    conv2d_direct_kernel<<<static_cast<unsigned>(blocks), 256, 0, a.stream>>>(
        X, Wt, Y, total, (int)H, (int)W, (int)C, (int)R, (int)S, (int)F, (int)a.OH, (int)a.OW,
        stride_h, stride_w, pad_top, pad_left, a.relu, a.thr);
    XTC_CUDA_CHECK(cudaGetLastError());
    return XTC_CUDA_OK;
  }
  XTC_REQUIRE(c.variant >= 0 && c.variant <= 5, "conv2d: unknown variant %d", c.variant);
  if (c.variant == 5) {
    const StreamPlan sp = plan_stream(a, c.tile_k == 16 ? 16 : 32);  // tile_k = 16: 16-channel slabs
    if (sp.ok) return launch_conv_stream(a, sp, workspace, workspace_bytes);
    set_error("conv2d: the streamed-weights variant (5) needs stride 1, channels and filters that are "
              "multiples of 4, 2 to 32 filter taps and two stages of one halo slab plus the taps' weights "
              "in shared memory");
    return XTC_CUDA_ERR_UNSUPPORTED;
  }
  if (c.variant == 4) {
    const SlidePlan sp = plan_slide(a);
    if (sp.ok) return sp.bn == 64 ? launch_conv_slide<64>(a, sp) : launch_conv_slide<128>(a, sp);
    set_error("conv2d: the sliding-window variant (4) needs stride 1, at most 128 filters, a halo run of "
              "at most 256 positions and a filter bank that fits beside five 16 KB ring slots");
    return XTC_CUDA_ERR_UNSUPPORTED;
  }
  if (c.variant == 3) {
    // Resident weights with two filter taps per MMA (only when asked for: see the numbers in
    // conv2d_halo_taps.cuh).
    HaloPlan t = plan_halo(a, false, 32, true);
    const HaloPlan t16 = plan_halo(a, false, 16, true);
    if (t16.ok && (c.tile_k == 16 || (c.tile_k != 32 && !t.ok))) t = t16;
    if (t.ok && c.tile_m != 2 * BM) return dispatch_conv_halo(a, t, false, true);
    set_error("conv2d: two taps per MMA (variant 3) needs stride 1, at most 64 filters, a filter row "
              "of two taps or more, one CTA per tile and a filter bank that fits in shared memory");
    return XTC_CUDA_ERR_UNSUPPORTED;
  }
  if (c.variant != 1) {
    // Resident weights + halo tiles: chosen when asked for, and by default when
    // the caller named no im2col-kernel parameter (pixel tile, K per stage).
    // One CTA per tile: 32-channel slabs unless two stages of them do not fit next to
    // the filter bank (measured on 32x56x56x64 -> 64, 3x3: five 16-channel stages are
    // no faster than two 32-channel ones, 24.1 vs 23.4 us).  tile_k = 16 or 32 forces it.
    HaloPlan h1 = plan_halo(a, false, 32);
    const HaloPlan h16 = plan_halo(a, false, 16);
    const bool narrow = c.tile_k == 16 || (c.tile_k != 32 && !h1.ok);
    if (narrow && h16.ok) h1 = h16;
    // nothing named and no room for the whole filter bank beside one CTA's stages: streamed
    // weights where that pays (stream_is_default), balanced over the pairs given the workspace
    if (c.variant == 0 && c.precision == XTC_CUDA_PRECISION_TF32 && c.tile_m == 0 && c.tile_n == 0 &&
        c.tile_k == 0 && c.split_k == 0 && !h1.ok) {
      const StreamPlan sp = plan_stream(a);
      if (stream_is_default(a, sp)) return launch_conv_stream(a, sp, workspace, workspace_bytes);
    }
    const HaloPlan h2 = plan_halo(a, true, 32);
    // the pair kernel when asked for (tile_m = 256) or when only half a filter bank fits
    const bool pair = c.tile_m == 2 * BM || (c.tile_m == 0 && !h1.ok && h2.ok);
    const HaloPlan& h = pair ? h2 : h1;
    const bool wanted = c.variant == 2 || (c.tile_m == 0 && c.tile_k == 0);
    if (h.ok && wanted) return dispatch_conv_halo(a, h, pair);
    if (c.variant == 2) {
      set_error("conv2d: the resident-weights variant needs stride 1 and a filter bank of at most "
                "%d bytes next to two halo stages (R*S*C*F too large here)", 232448 - 2048);
      return XTC_CUDA_ERR_UNSUPPORTED;
    }
  }
  XTC_REQUIRE(c.tile_m == 0 || c.tile_m == BM || c.tile_m == 2 * BM,
              "conv2d: tile_m=%d unsupported (128, or 256 for the CTA-pair kernel)", c.tile_m);
  int tile_m = c.tile_m, tile_n = c.tile_n;
  if (tile_m == 0 && tile_n == 0 && c.tile_k == 0) {
    // nothing named: the GEMM cost model on M = pixels, N = filters, K = taps x padded channels
    // (split-K only with the zeroed workspace xtc_cuda_conv2d_workspace_bytes asks for)
    const int64_t kpad = R * S * ((C + 31) / 32 * 32);
    int caps[9] = {};
    for (int sz = 2; sz <= 8; ++sz) caps[sz] = cluster_capacity(dev, sz);
    AutoChoice pick = choose_tf32_default(M, F, kpad, sm_count(dev), a16(Y), true,
                                          a16(Y) && F % 4 == 0 ? caps : nullptr, false);
    const size_t need = conv_split_bytes(M, F, pick);
    if (need > 0 && c.split_k == 0 && a16(Y) && conv_split_in_cluster(M, F, pick, dev)) {
      a.split_k = pick.split_k;
      a.cluster_k = true;
    } else if (need > 0 && c.split_k == 0 && workspace != nullptr && workspace_bytes >= need) {
      const size_t tiles = static_cast<size_t>((M + BM - 1) / BM) * ((F + pick.tile_n - 1) / pick.tile_n);
      a.split_k = pick.split_k;
      a.counters = static_cast<int*>(workspace);
      a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                            ((tiles * 4 + 255) & ~static_cast<size_t>(255)));
    } else if (need > 0) {
      pick = choose_tf32_default(M, F, kpad, sm_count(dev), a16(Y), false, nullptr, false);
    }
    tile_m = pick.tile_m;
    tile_n = pick.tile_n;
    // One round of tiles either way: the one-CTA kernel.  A pair halves the filter loads but
    // not the im2col loads, and its hand-offs cost more than that saves (14x14x256 -> 256:
    // 21.5 us against 22.4 us; 28x28x128 -> 256 stride 2: 13.3 us against 14.6 us).
    if (tile_m == 2 * BM && ((M + BM - 1) / BM) * ((F + tile_n - 1) / tile_n) <= sm_count(dev))
      tile_m = BM;
  }
  if (tile_n == 0) tile_n = F <= 64 ? 64 : (F <= 128 ? 128 : 256);
  if (c.split_k > 1 && tile_m != 2 * BM && a16(Y)) {
    // a split the caller asked for runs where the cluster form applies, else the layer runs unsplit
    const AutoChoice asked{BM, tile_n, 0, c.split_k};
    if (conv_split_in_cluster(M, F, asked, dev)) {
      a.split_k = c.split_k;
      a.cluster_k = true;
    }
  }
  int tile_k = c.tile_k ? c.tile_k : (C % 64 == 0 ? 64 : 32);
  // bulk tensor stores unless direct stores were asked for (14x14x256 -> 256: 21.5 us against 23.1 us)
  const bool tma_store = (c.epilogue == 2 || (c.epilogue == 0 && !a.cluster_k)) && a16(Y) && F % 4 == 0;
  if (tile_m == 2 * BM && a16(Y)) return dispatch_conv_pair(a, tile_n, tile_k);
  return tma_store ? dispatch_conv<true>(a, tile_n, tile_k) : dispatch_conv<false>(a, tile_n, tile_k);
}
