// TF32 tensor-core GEMM for sm_100a: C[M,N] = A[M,K] * B[K,N] (+ relu).
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer   (global -> swizzled shared-memory ring)
//   warp 1      MMA issuer     (tcgen05.mma kind::tf32, accumulators in TMEM)
//   warps 2..5  epilogue       (tcgen05.ld -> relu -> global / TMA store)
// The accumulator is double buffered in TMEM so the epilogue of one output
// tile overlaps the main loop of the next.
//
// Operand layouts in shared memory
//   K-major operand (A stored [M,K], or B stored [N,K]): 128-byte rows of 32
//     floats along K, SWIZZLE_128B, 8-row groups 1024 bytes apart.
//   MN-major operand (B stored [K,N], or A stored [K,M]): 128-byte rows of 32
//     floats along M/N, one row per k, SWIZZLE_128B with 32-byte atoms (the
//     only swizzle the tensor core accepts for transposed 32-bit operands),
//     4-row groups 512 bytes apart, 32-column groups BK*128 bytes apart.
#pragma once
#include "common.cuh"

namespace xtc {

using namespace dev;

static constexpr int BM = 128;         // UMMA M (cta_group::1)
static constexpr int NUM_THREADS = 192;
static constexpr int EPI_WARPS = 4;

// How the A operand reaches shared memory.
enum : int {
  A_KMAJOR = 0,  // A stored [M,K] row-major: 2-D tiled TMA, K-major UMMA operand
  A_MNMAJOR = 1, // A stored [K,M] row-major (a fused transpose): MN-major UMMA operand
  A_IM2COL = 2   // A is the implicit im2col matrix of an NHWC tensor: im2col-mode TMA
};

struct GemmParams {
  float* C;
  int64_t ldc;
  int M, N, K;
  int tiles_m, tiles_n, k_blocks;
  int group_n;        // tile columns per panel of the tile order (0 = 4), see tile_coords
  int chunk_kblocks;  // K stages accumulated in one TMEM buffer before the epilogue takes it
  int relu;
  float relu_threshold;
  int* status;
  // implicit-GEMM convolution (A_IM2COL): row m = (image, oh, ow), k = (r, s, c)
  int conv_ohow, conv_ow, conv_c, conv_cblocks, conv_s;
  int conv_stride_h, conv_stride_w, conv_pad_top, conv_pad_left;
  // Broadcast epilogue: every output tile is also written, with plain coalesced
  // stores, to the same position of up to 7 more buffers (the copies of C that
  // peer GPUs hold, mapped into this process), fusing the all-gather of a
  // row-sharded matmul into the GEMM.
  int n_extra;
  float* extra_dst[7];
  // The same broadcast through an NVLink multicast mapping (CTA-pair kernel, copier warps):
  // mc_dst addresses this rank's block of C in a multicast object that every rank's C is
  // bound to, so ONE multimem.st per vector reaches every GPU (the NVSwitch replicates it)
  // where the unicast form issues one store per peer.  NULL = unicast stores to extra_dst.
  float* mc_dst;
  // CTA-pair kernel: the TMA stores of C carry an L2 evict-first hint, so that the output
  // passing through L2 pushes out as little of the operand panels the wave still re-reads
  // as possible.  Off when copier warps read the finished tiles back from L2.
  int c_evict_first;
  // Split-K (small problems with fewer tiles than SMs): `split_k` CTAs share one
  // output tile, each over `split_kblocks` K stages.  Every CTA writes its raw
  // partial tile to `partials` [split][tile][128][BN]; the last one to arrive on
  // `tile_counters[tile]` sums the partials in split order (deterministic),
  // applies the epilogue and resets the counter.
  int split_k;
  int split_kblocks;
  float* partials;
  int* tile_counters;
  // Split-K inside a thread-block cluster (cluster_k = 1; split_k is the cluster size,
  // 2 to 8; one work item per CTA): the CTAs of a cluster hold the K pieces of one
  // tile, park their accumulators in their own shared memory (the operand ring is free
  // by then) and each sums ceil(128 / split_k) rows of the tile over all pieces through
  // distributed shared memory, in piece order.  No workspace, no pass through L2.
  int cluster_k;
  // Split tail of the CTA-pair kernel (gemm_tf32_pair.cuh): the tail_tiles tiles of
  // the last, partly idle round are each cut into tail_split pieces along K, one
  // piece per pair.  tail_split = 0 turns it off.
  int tail_first;      // index of the first tail tile (= tiles - tail_tiles)
  int tail_tiles;
  int tail_split;
  int* sk_flags;       // [tail tile][piece - 1][8 slabs]: "parked" flags (zeroed once)
  float* sk_partials;  // [tail tile][piece - 1][8 slabs][32 x BN] raw accumulators
};

template <int BN, int KSPANS, bool SPLIT3>
struct SmemLayout {
  static constexpr int BK = 32 * KSPANS;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int OPERANDS = SPLIT3 ? 2 : 1;
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * OPERANDS;
  // Per epilogue warp, two 32x32 fp32 staging tiles for TMA stores.
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * 32 * 32 * 4;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int max_stages(bool tma_store) {
    int avail = 232448 - 1024 /*alignment slack*/ - BAR_BYTES - (tma_store ? EPI_BYTES : 0);
    int s = avail / STAGE_BYTES;
    return s > 8 ? 8 : s;
  }
  static constexpr int total(int stages, bool tma_store) {
    return 1024 + BAR_BYTES + (tma_store ? EPI_BYTES : 0) + stages * STAGE_BYTES;
  }
};

// tile index -> (m, n) tile coordinates.  Tiles are walked in panels of group_n tile
// columns, columns fastest inside a panel, so that the tiles in flight at one time (one per
// SM or SM pair) form a near-square block: its A rows and B columns are then the smallest
// operand set L2 has to keep for that wave (panel_columns() picks group_n on the host).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_n, int& tm,
                                            int& tn) {
  const int gw = group_n > 0 ? group_n : 4;
  int per_group = tiles_m * gw;
  int g = tile / per_group;
  int first_n = g * gw;
  int gn = min(gw, tiles_n - first_n);
  int r = tile - g * per_group;
  tm = r / gn;
  tn = first_n + (r - tm * gn);
}

// Panel width for `slots` tiles in flight of tile_rows x tile_cols outputs: the width w that
// minimises the operand bytes of a wave, w * tile_cols + (slots / w) * tile_rows (both times K).
inline int panel_columns(int slots, int tile_rows, int tile_cols, int tiles_n) {
  int best = 1;
  double best_cost = 1e300;
  for (int w = 1; w <= tiles_n && w <= slots; ++w) {
    const double rows = static_cast<double>(slots) / w;
    const double cost = static_cast<double>(w) * tile_cols + rows * tile_rows;
    if (cost < best_cost) { best_cost = cost; best = w; }
  }
  return best;
}

template <int BN, int KSPANS, int A_MODE, bool B_MN, bool SPLIT3, bool TMA_STORE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmAlo,
                 const __grid_constant__ CUtensorMap tmBlo,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p, const int stages) {
  using L = SmemLayout<BN, KSPANS, SPLIT3>;
  constexpr int BK = L::BK;
  constexpr bool A_MN = A_MODE == A_MNMAJOR;
  static_assert(!(A_MODE == A_IM2COL && SPLIT3), "the 3xTF32 split is not wired for im2col loads");
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* ring = smem;  // stages * STAGE_BYTES, 1024-aligned
  uint8_t* epi = ring + static_cast<size_t>(stages) * L::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + (TMA_STORE ? L::EPI_BYTES : 0));
  uint64_t* full = bars;             // [stages]
  uint64_t* empty = bars + 8;        // [stages]
  uint64_t* acc_full = bars + 16;    // [2]
  uint64_t* acc_empty = bars + 18;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (SPLIT3) {
      prefetch_tmap(&tmAlo);
      prefetch_tmap(&tmBlo);
    }
    if (TMA_STORE) prefetch_tmap(&tmC);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dependency_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Work items: (tile, K split).  Without split-K there is one item per tile.
  const int real_tiles = p.tiles_m * p.tiles_n;
  const int num_tiles = real_tiles * p.split_k;
  bool failed = false;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int item = blockIdx.x; item < num_tiles && !failed; item += gridDim.x) {
        const int tile = item / p.split_k;
        const int kb_lo = (item - tile * p.split_k) * p.split_kblocks;
        const int kb_hi = min(kb_lo + p.split_kblocks, p.k_blocks);
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        int img = 0, ih0 = 0, iw0 = 0;  // input pixel under the filter origin of row m0
        if (A_MODE == A_IM2COL) {
          img = m0 / p.conv_ohow;
          const int rem = m0 - img * p.conv_ohow;
          const int oh = rem / p.conv_ow;
          ih0 = oh * p.conv_stride_h - p.conv_pad_top;
          iw0 = (rem - oh * p.conv_ow) * p.conv_stride_w - p.conv_pad_left;
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_EMPTY);
            failed = true;
            break;
          }
          uint8_t* sA = ring + static_cast<size_t>(stage) * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          mbar_arrive_expect_tx(&full[stage], L::STAGE_BYTES);
          int k0 = kb * BK;
          int fr = 0, fs = 0, c0 = 0;  // filter tap and first channel of this K block
          if (A_MODE == A_IM2COL) {
            const int rs = kb / p.conv_cblocks;
            c0 = (kb - rs * p.conv_cblocks) * BK;
            fr = rs / p.conv_s;
            fs = rs - fr * p.conv_s;
            k0 = rs * p.conv_c + c0;
          }
#pragma unroll
          for (int op = 0; op < L::OPERANDS; ++op) {
            const CUtensorMap* ta = op == 0 ? &tmA : &tmAlo;
            const CUtensorMap* tb = op == 0 ? &tmB : &tmBlo;
            uint8_t* dA = sA + op * (L::A_BYTES + L::B_BYTES);
            uint8_t* dB = sB + op * (L::A_BYTES + L::B_BYTES);
            if (A_MODE == A_IM2COL) {
#pragma unroll
              for (int s = 0; s < KSPANS; ++s)
                tma_load_im2col_4d(dA + s * (BM * 128), ta, &full[stage], c0 + s * 32, iw0, ih0,
                                   img, static_cast<uint16_t>(fs), static_cast<uint16_t>(fr));
            } else if (A_MODE == A_KMAJOR) {
#pragma unroll
              for (int s = 0; s < KSPANS; ++s)
                tma_load_2d(dA + s * (BM * 128), ta, &full[stage], k0 + s * 32, m0);
            } else {
#pragma unroll
              for (int g = 0; g < BM / 32; ++g)
                tma_load_2d(dA + g * (BK * 128), ta, &full[stage], m0 + g * 32, k0);
            }
            if (B_MN) {
#pragma unroll
              for (int g = 0; g < BN / 32; ++g)
                tma_load_2d(dB + g * (BK * 128), tb, &full[stage], n0 + g * 32, k0);
            } else {
#pragma unroll
              for (int s = 0; s < KSPANS; ++s)
                tma_load_2d(dB + s * (BN * 128), tb, &full[stage], k0 + s * 32, n0);
            }
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The K loop of a tile is cut into chunks of p.chunk_kblocks stages; each
    // chunk accumulates into the next TMEM buffer and is handed to the epilogue.
    // The TF32 mode uses one chunk per tile.  The 3xTF32 mode uses short chunks
    // that the epilogue sums in fp32 registers: the tensor core truncates when it
    // adds into its accumulator, and a short chain keeps that error below 1e-5.
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc_iter = 0;
      for (int item = blockIdx.x; item < num_tiles && !failed; item += gridDim.x) {
        const int kb_lo = (item % p.split_k) * p.split_kblocks;
        const int kb_hi = min(kb_lo + p.split_kblocks, p.k_blocks);
        for (int kb0 = kb_lo; kb0 < kb_hi && !failed; kb0 += p.chunk_kblocks, ++acc_iter) {
          const int acc = acc_iter & 1;
          const uint32_t acc_phase = (acc_iter >> 1) & 1;
          if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_DRAIN);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          const int kb_end = min(kb0 + p.chunk_kblocks, kb_hi);
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!mbar_wait(&full[stage], phase)) {
              atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
              failed = true;
              break;
            }
            tc_fence_after();
            const uint32_t sA = smem_u32(ring + static_cast<size_t>(stage) * L::STAGE_BYTES);
            const uint32_t sB = sA + L::A_BYTES;
            // descriptor halves once per stage; per MMA only the low half moves
            const uint32_t a_hi = A_MN ? umma_desc_hi(512, (uint32_t)UMMA_SWIZZLE_128B_BASE32B)
                                       : umma_desc_hi(1024, (uint32_t)UMMA_SWIZZLE_128B);
            const uint32_t b_hi = B_MN ? umma_desc_hi(512, (uint32_t)UMMA_SWIZZLE_128B_BASE32B)
                                       : umma_desc_hi(1024, (uint32_t)UMMA_SWIZZLE_128B);
            const uint32_t a_lo = umma_desc_lo(sA, A_MN ? BK * 128 : 16);
            const uint32_t b_lo = umma_desc_lo(sB, B_MN ? BK * 128 : 16);
            const uint32_t first = kb > kb0 ? 1u : 0u;
#pragma unroll
            for (int kk = 0; kk < BK / 8; ++kk) {
              // byte offsets of K step kk inside the stage, >> 4
              const uint32_t aoff =
                  (A_MN ? kk * 1024 : (kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
              const uint32_t boff =
                  (B_MN ? kk * 1024 : (kk >> 2) * (BN * 128) + (kk & 3) * 32) >> 4;
              const uint32_t acc_in = first | (kk != 0);
              if (!SPLIT3) {
                umma_tf32(d_tmem, umma_desc_pack(a_lo + aoff, a_hi),
                          umma_desc_pack(b_lo + boff, b_hi), idesc, acc_in);
              } else {
                constexpr uint32_t lo = (L::A_BYTES + L::B_BYTES) >> 4;  // the lo-part tiles
                // small cross terms first, the dominant hi*hi product last
                umma_tf32(d_tmem, umma_desc_pack(a_lo + lo + aoff, a_hi),
                          umma_desc_pack(b_lo + boff, b_hi), idesc, acc_in);
                umma_tf32(d_tmem, umma_desc_pack(a_lo + aoff, a_hi),
                          umma_desc_pack(b_lo + lo + boff, b_hi), idesc, 1);
                umma_tf32(d_tmem, umma_desc_pack(a_lo + aoff, a_hi),
                          umma_desc_pack(b_lo + boff, b_hi), idesc, 1);
              }
            }
            tc_commit(&empty[stage]);  // stage reusable once these MMAs retire
            if (++stage == stages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (!failed) tc_commit(&acc_full[acc]);
        }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int epi_id = warp - 2;
    float* stage_buf = reinterpret_cast<float*>(epi + epi_id * (2 * 32 * 32 * 4));
    int acc_iter = 0;
    int buf = 0;
    const bool vec_ok = (p.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;

    // relu + store of one 32-row x 32-column block held one row per lane
    auto store_block = [&](uint32_t (&r)[32], int m0, int col0) {
      if (p.relu) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          r[i] = __float_as_uint(fmaxf(__uint_as_float(r[i]), p.relu_threshold));
      }
      if (TMA_STORE) {
        // Stage the block in shared memory with the 128-byte swizzle the store's
        // tensor map expects, then one lane issues the bulk store.
        float* sb = stage_buf + buf * (32 * 32);
        tma_store_wait_read<1>();  // the buffer used two stores ago is free
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int chunk = j ^ (lane & 7);
          float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          *reinterpret_cast<float4*>(sb + lane * 32 + chunk * 4) = v;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && col0 < p.N && m0 + quad * 32 < p.M)
          tma_store_2d(&tmC, sb, col0, m0 + quad * 32);
        if (lane == 0) tma_store_commit();
        if (p.n_extra > 0) {
          // Read the staged block back row-wise: 8 lanes cover one 128-byte row, so a
          // warp-wide store writes four full rows -- whole 128-byte lines on the link.
          const int chunk = lane & 7;
          const int gcol = col0 + chunk * 4;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r_in = i * 4 + (lane >> 3);
            const int grow = m0 + quad * 32 + r_in;
            const float4 v =
                *reinterpret_cast<const float4*>(sb + r_in * 32 + ((chunk ^ (r_in & 7)) << 2));
            if (grow < p.M && gcol < p.N) {
              const int64_t off = static_cast<int64_t>(grow) * p.ldc + gcol;
              for (int d = 0; d < p.n_extra; ++d)
                *reinterpret_cast<float4*>(p.extra_dst[d] + off) = v;
            }
          }
        }
        buf ^= 1;
      } else {
        const int row = m0 + quad * 32 + lane;
        if (row < p.M) {
          float* dst = p.C + static_cast<int64_t>(row) * p.ldc + col0;
          if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
              reinterpret_cast<float4*>(dst)[j] = v;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.N) dst[i] = __uint_as_float(r[i]);
          }
        }
      }
    };

    const bool split = !SPLIT3 && p.split_k > 1;
    uint32_t* last_flag = tmem_slot + 1;  // written by one epilogue thread, read by all 128
    for (int item = blockIdx.x; item < num_tiles && !failed; item += gridDim.x) {
      const int tile = item / p.split_k;
      const int my_split = item - tile * p.split_k;
      const int kb_lo = my_split * p.split_kblocks;
      const int kb_hi = min(kb_lo + p.split_kblocks, p.k_blocks);
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      float sum[SPLIT3 ? BN : 1];
      if (SPLIT3) {
#pragma unroll
        for (int i = 0; i < (SPLIT3 ? BN : 1); ++i) sum[i] = 0.f;
      }
      // this thread's row of the partial tile [split][tile][128][BN]
      float* part_row = nullptr;
      if (split)
        part_row = p.partials +
                   ((static_cast<size_t>(my_split) * real_tiles + tile) * BM + quad * 32 + lane) * BN;
      for (int kb0 = kb_lo; kb0 < kb_hi && !failed; kb0 += p.chunk_kblocks, ++acc_iter) {
        const int acc = acc_iter & 1;
        const uint32_t acc_phase = (acc_iter >> 1) & 1;
        if (!mbar_wait(&acc_full[acc], acc_phase)) {
          if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
          failed = true;
          break;
        }
        tc_fence_after();
        if (SPLIT3) {
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + lane_base + acc * BN + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) sum[(SPLIT3 ? c * 32 : 0) + (SPLIT3 ? i : 0)] += __uint_as_float(r[i]);
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + lane_base + acc * BN + c * 32, r);
            tmem_ld_wait();
            if (!split) {
              store_block(r, m0, n0 + c * 32);
            } else if (p.cluster_k) {
              // float4 (row, q) of the tile lives at [q][row]: a warp writes 512 contiguous bytes
              float4* red4 = reinterpret_cast<float4*>(ring);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                red4[(c * 8 + j) * BM + quad * 32 + lane] =
                    make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                __stcg(reinterpret_cast<float4*>(part_row + c * 32) + j,
                       make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                   __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
            }
          }
        }
        // all TMEM reads of this warp are complete (wait::ld above): release the buffer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
      }
      if (SPLIT3 && !failed) {
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(sum[(SPLIT3 ? c * 32 : 0) + (SPLIT3 ? i : 0)]);
          store_block(r, m0, n0 + c * 32);
        }
      }
      if (split && !p.cluster_k && !failed) {
        // Publish the partial, count arrivals; the CTA that completes the tile reduces.
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const int old = atomicAdd(&p.tile_counters[tile], 1);
          *last_flag = (old == p.split_k - 1) ? 1u : 0u;
          if (old == p.split_k - 1) p.tile_counters[tile] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = *reinterpret_cast<volatile uint32_t*>(last_flag) != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");  // flag read by all before it is rewritten
        if (last) {
          __threadfence();
          const size_t split_stride = static_cast<size_t>(real_tiles) * BM * BN;
          const float* row0 = p.partials + (static_cast<size_t>(tile) * BM + quad * 32 + lane) * BN;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            float4 accv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) accv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < p.split_k; ++s) {  // fixed order: bit-reproducible
              const float4* src = reinterpret_cast<const float4*>(row0 + s * split_stride + c * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 v = __ldcg(src + j);
                accv[j].x += v.x; accv[j].y += v.y; accv[j].z += v.z; accv[j].w += v.w;
              }
            }
            uint32_t r[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              r[4 * j] = __float_as_uint(accv[j].x); r[4 * j + 1] = __float_as_uint(accv[j].y);
              r[4 * j + 2] = __float_as_uint(accv[j].z); r[4 * j + 3] = __float_as_uint(accv[j].w);
            }
            store_block(r, m0, n0 + c * 32);
          }
        }
      }
    }
    if (TMA_STORE) tma_store_wait_all<0>();
  }

  if (p.cluster_k) {
    // Every thread of the cluster meets here twice, whatever its role did before (the
    // role loops above are bounded, so a CTA whose wait gave up still arrives).
    __syncwarp();
    cluster_sync_all();  // all pieces of the tile are parked in their CTAs' shared memory
    if (warp >= 2) {
      const int tile = static_cast<int>(blockIdx.x) / p.split_k;
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int rows_own = (BM + p.split_k - 1) / p.split_k;  // the last piece may own fewer
      const int rank = static_cast<int>(cluster_ctarank());  // = this CTA's piece
      const uint32_t red_base = smem_u32(ring);
      // Two float4 of the tile per thread and round, all their pieces requested before the first
      // is added: a remote shared-memory read is a round trip of several hundred clocks, and a
      // loop that waits for each one in turn spent 2 us on the 16 reads a thread makes for c1.
      const int total = rows_own * (BN / 4);
      constexpr int STRIDE = EPI_WARPS * 32;
      for (int i = (warp - 2) * 32 + lane; i < total; i += 2 * STRIDE) {
        // items ia and ib; a row past the tile (128 does not divide by 3, 5, 6 or 7) or the
        // missing partner of a last odd round is replaced by the other item, whose store
        // then happens once
        int ia = i, ib = i + STRIDE < total ? i + STRIDE : i;
        const bool ok_a = rank * rows_own + ia % rows_own < BM;
        const bool ok_b = rank * rows_own + ib % rows_own < BM;
        if (!ok_a && !ok_b) continue;
        if (!ok_a) ia = ib;
        if (!ok_b) ib = ia;
        const int qa = ia / rows_own, qb = ib / rows_own;
        const int row_a = rank * rows_own + (ia - qa * rows_own);
        const int row_b = rank * rows_own + (ib - qb * rows_own);
        const uint32_t addr_a = red_base + static_cast<uint32_t>(qa * BM + row_a) * 16u;
        const uint32_t addr_b = red_base + static_cast<uint32_t>(qb * BM + row_b) * 16u;
        float4 acc_a, acc_b;
        switch (p.split_k) {  // fixed piece order: bit-reproducible
          case 2: sum_cluster_pieces<2>(addr_a, addr_b, acc_a, acc_b); break;
          case 3: sum_cluster_pieces<3>(addr_a, addr_b, acc_a, acc_b); break;
          case 4: sum_cluster_pieces<4>(addr_a, addr_b, acc_a, acc_b); break;
          case 5: sum_cluster_pieces<5>(addr_a, addr_b, acc_a, acc_b); break;
          case 6: sum_cluster_pieces<6>(addr_a, addr_b, acc_a, acc_b); break;
          case 7: sum_cluster_pieces<7>(addr_a, addr_b, acc_a, acc_b); break;
          default: sum_cluster_pieces<8>(addr_a, addr_b, acc_a, acc_b); break;
        }
        if (p.relu) {
          acc_a.x = fmaxf(acc_a.x, p.relu_threshold); acc_a.y = fmaxf(acc_a.y, p.relu_threshold);
          acc_a.z = fmaxf(acc_a.z, p.relu_threshold); acc_a.w = fmaxf(acc_a.w, p.relu_threshold);
          acc_b.x = fmaxf(acc_b.x, p.relu_threshold); acc_b.y = fmaxf(acc_b.y, p.relu_threshold);
          acc_b.z = fmaxf(acc_b.z, p.relu_threshold); acc_b.w = fmaxf(acc_b.w, p.relu_threshold);
        }
        const int grow_a = m0 + row_a, gcol_a = n0 + 4 * qa;
        if (grow_a < p.M && gcol_a < p.N)  // N is a multiple of 4 in this mode
          *reinterpret_cast<float4*>(p.C + static_cast<size_t>(grow_a) * p.ldc + gcol_a) = acc_a;
        const int grow_b = m0 + row_b, gcol_b = n0 + 4 * qb;
        if (ib != ia && grow_b < p.M && gcol_b < p.N)
          *reinterpret_cast<float4*>(p.C + static_cast<size_t>(grow_b) * p.ldc + gcol_b) = acc_b;
      }
    }
    __syncwarp();
    cluster_sync_all();  // no CTA leaves while the others still read its shared memory
  }

  if (failed) {
    // Unwind path of a bounded wait that gave up: give copies that may still be
    // in flight towards this CTA's shared memory time to land before exiting.
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace xtc
