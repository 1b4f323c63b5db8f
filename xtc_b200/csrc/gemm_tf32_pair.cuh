// TF32 GEMM on CTA pairs (tcgen05 cta_group::2): two SMs share one 256 x BN MMA.
//
// Each CTA of a 2-CTA cluster loads its own 128 rows of A and its own half of
// the B tile (BN/2 columns), so per SM the shared-memory traffic for B halves
// compared with the single-CTA kernel, which is what limits that kernel.  The
// even CTA (the leader) issues the MMAs for both; each CTA's 128 x BN slice of
// the accumulator lives in its own TMEM and is drained by its own epilogue.
//
// Synchronisation across the pair (no multicast anywhere):
//   full[s]      leader only.  Both producers' TMA loads report their bytes to it.
//   empty[s]     one per CTA.  The leader commits to both after the MMAs of a stage.
//   acc_full[a]  one per CTA.  The leader commits to both after the last MMA of a tile.
//   acc_empty[a] leader only, 8 arrivals: the 4 epilogue warps of both CTAs.
//
// Split tail.  With T tiles on P pairs the last of ceil(T/P) rounds is partly idle
// (4096^3: 256 tiles on 74 pairs, 3.46 rounds of work in 4).  When the launcher
// provides a workspace and the rem = T mod P tiles of the last round number at
// most P/2, each of them is cut into S = floor(P/rem) pieces along K and every
// piece goes to a pair of its own, so the last round lasts 1/S as long.  Pieces
// 1..S-1 park their raw accumulators in the workspace; the pair that holds piece
// 0 waits for them, adds them to its own in piece order (so the result does not
// depend on timing) and stores the tile.  All pieces of a round start together,
// so tiles that share an operand panel still stream it in step and L2 serves the
// re-reads; cutting K into contiguous per-pair ranges instead (stream-K) was
// measured slower than no split at all for that reason (4096^3: 210 us against
// 198 us; 8192x1024x8192: 278 us against 190 us).
#pragma once
#include "gemm_tf32.cuh"

namespace xtc {

struct PairWork {
  int tile, kb0, kb1;
  int piece;  // 0 = this pair stores the tile; > 0 = it parks its accumulator
  int split;  // pieces the tile is cut into (1 = whole tile)
  int tail;   // index of the tile among the tail tiles
};

// The sequence of work items of one pair; the producer, the MMA issuer and the
// epilogue warps each walk their own copy.
struct PairWorkIter {
  int next_tile, stride, pair;
  bool tail_done;
  __device__ PairWorkIter(int pair_, int num_pairs)
      : next_tile(pair_), stride(num_pairs), pair(pair_), tail_done(false) {}
  __device__ bool next(const GemmParams& p, PairWork& w) {
    const int whole = p.tail_split > 0 ? p.tail_first : p.tiles_m * p.tiles_n;
    if (next_tile < whole) {
      w.tile = next_tile;
      w.kb0 = 0;
      w.kb1 = p.k_blocks;
      w.piece = 0;
      w.split = 1;
      w.tail = 0;
      next_tile += stride;
      return true;
    }
    if (p.tail_split > 0 && !tail_done && pair < p.tail_tiles * p.tail_split) {
      tail_done = true;
      w.tail = pair / p.tail_split;
      w.piece = pair - w.tail * p.tail_split;
      w.split = p.tail_split;
      w.tile = p.tail_first + w.tail;
      w.kb0 = static_cast<int>(static_cast<long long>(p.k_blocks) * w.piece / p.tail_split);
      w.kb1 = static_cast<int>(static_cast<long long>(p.k_blocks) * (w.piece + 1) / p.tail_split);
      return true;
    }
    return false;
  }
};

template <int BN, int KSPANS>
struct PairSmem {
  static constexpr int BK = 32 * KSPANS;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = (BN / 2) * BK * 4;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = EPI_WARPS * 2 * 32 * 32 * 4;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int max_stages() {
    int s = (232448 - 1024 - BAR_BYTES - EPI_BYTES) / STAGE_BYTES;
    return s > 8 ? 8 : s;
  }
  static constexpr int total(int stages) { return 1024 + BAR_BYTES + EPI_BYTES + stages * STAGE_BYTES; }
};

// Threads per CTA: the six warps of gemm_tf32.cuh, plus four copier warps when the
// output is also broadcast to peer GPUs (launched only then).
constexpr int PAIR_THREADS = NUM_THREADS;
constexpr int PAIR_THREADS_BCAST = NUM_THREADS + 4 * 32;

template <int BN, int KSPANS, int A_MODE, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS_BCAST, 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const GemmParams p,
                      const int stages) {
  using L = PairSmem<BN, KSPANS>;
  constexpr int BK = L::BK;
  constexpr bool A_MN = A_MODE == A_MNMAJOR;
  constexpr int HALF = BN / 2;
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* ring = smem;
  uint8_t* epi = ring + static_cast<size_t>(stages) * L::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + L::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + 8;
  uint64_t* acc_full = bars + 16;
  uint64_t* acc_empty = bars + 18;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  // tiles stored so far by the epilogue warp of each TMEM quadrant (read by its copier warp)
  volatile uint32_t* stored = reinterpret_cast<volatile uint32_t*>(bars + 24);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  // Broadcast with copier warps: the epilogue only stores the tile locally and counts
  // it; warps 6..9 copy finished tiles from the local C to the peers, so the tensor
  // pipeline never waits for NVLink.
  const bool copiers = (p.n_extra > 0 || p.mc_dst != nullptr) && blockDim.x > PAIR_THREADS;

  if (threadIdx.x == 0) {
    for (int q = 0; q < 4; ++q) stored[q] = 0;
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmC);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers exist before anything signals them
  tc_fence_after();
  grid_dependency_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  bool failed = false;

  if (warp == 0) {
    // ---------------------- TMA producer (one per CTA) ------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      PairWorkIter work(pair, num_pairs);
      PairWork w;
      while (!failed && work.next(p, w)) {
        int tm, tn;
        tile_coords(w.tile, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
        const int m0 = tm * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * HALF;
        int img = 0, ih0 = 0, iw0 = 0;  // input pixel under the filter origin of row m0
        if (A_MODE == A_IM2COL) {
          img = m0 / p.conv_ohow;
          const int rem = m0 - img * p.conv_ohow;
          const int oh = rem / p.conv_ow;
          ih0 = oh * p.conv_stride_h - p.conv_pad_top;
          iw0 = (rem - oh * p.conv_ow) * p.conv_stride_w - p.conv_pad_left;
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_EMPTY);
            failed = true;
            break;
          }
          uint8_t* sA = ring + static_cast<size_t>(stage) * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          if (leader) mbar_arrive_expect_tx(&full[stage], 2 * L::STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          int k0 = kb * BK;
          if (A_MODE == A_IM2COL) {
            const int rs = kb / p.conv_cblocks;
            const int c0 = (kb - rs * p.conv_cblocks) * BK;
            const int fr = rs / p.conv_s;
            const int fs = rs - fr * p.conv_s;
            k0 = rs * p.conv_c + c0;
#pragma unroll
            for (int s = 0; s < KSPANS; ++s)
              tma_load_im2col_4d_pair(sA + s * (BM * 128), &tmA, bar, c0 + s * 32, iw0, ih0, img,
                                      static_cast<uint16_t>(fs), static_cast<uint16_t>(fr));
          } else if (A_MODE == A_KMAJOR) {
#pragma unroll
            for (int s = 0; s < KSPANS; ++s)
              tma_load_2d_pair(sA + s * (BM * 128), &tmA, bar, k0 + s * 32, m0);
          } else {
#pragma unroll
            for (int g = 0; g < BM / 32; ++g)
              tma_load_2d_pair(sA + g * (BK * 128), &tmA, bar, m0 + g * 32, k0);
          }
          if (B_MN) {
#pragma unroll
            for (int g = 0; g < HALF / 32; ++g)
              tma_load_2d_pair(sB + g * (BK * 128), &tmB, bar, n0 + g * 32, k0);
          } else {
#pragma unroll
            for (int s = 0; s < KSPANS; ++s)
              tma_load_2d_pair(sB + s * (HALF * 128), &tmB, bar, k0 + s * 32, n0);
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------ MMA issuer (leader CTA) -------------------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_tf32(2 * BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      PairWorkIter work(pair, num_pairs);
      PairWork w;
      for (; !failed && work.next(p, w); ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_DRAIN);
          failed = true;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(ring + static_cast<size_t>(stage) * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
          const uint32_t a_hi = A_MN ? umma_desc_hi(512, (uint32_t)UMMA_SWIZZLE_128B_BASE32B)
                                     : umma_desc_hi(1024, (uint32_t)UMMA_SWIZZLE_128B);
          const uint32_t b_hi = B_MN ? umma_desc_hi(512, (uint32_t)UMMA_SWIZZLE_128B_BASE32B)
                                     : umma_desc_hi(1024, (uint32_t)UMMA_SWIZZLE_128B);
          const uint32_t a_lo = umma_desc_lo(sA, A_MN ? BK * 128 : 16);
          const uint32_t b_lo = umma_desc_lo(sB, B_MN ? BK * 128 : 16);
          const uint32_t first = kb != w.kb0 ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < BK / 8; ++kk) {
            const uint32_t aoff = (A_MN ? kk * 1024 : (kk >> 2) * (BM * 128) + (kk & 3) * 32) >> 4;
            const uint32_t boff =
                (B_MN ? kk * 1024 : (kk >> 2) * (HALF * 128) + (kk & 3) * 32) >> 4;
            umma_tf32_pair(d_tmem, umma_desc_pack(a_lo + aoff, a_hi),
                           umma_desc_pack(b_lo + boff, b_hi), idesc, first | (kk != 0));
          }
          // both CTAs may refill this stage once the MMAs above have read it
          const uint32_t e = smem_u32(&empty[stage]);
          tc_commit_pair(map_to_cta(e, 0));
          tc_commit_pair(map_to_cta(e, 1));
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!failed) {
          const uint32_t f = smem_u32(&acc_full[acc]);
          tc_commit_pair(map_to_cta(f, 0));
          tc_commit_pair(map_to_cta(f, 1));
        }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------- epilogue (both CTAs) ---------------------------
    const int quad = warp & 3;
    const int epi_id = warp - 2;
    float* stage_buf = reinterpret_cast<float*>(epi + epi_id * (2 * 32 * 32 * 4));
    const uint64_t store_policy = l2_policy_evict_first();
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int local = 0;
    int buf = 0;
    PairWorkIter work(pair, num_pairs);
    PairWork w;
    for (; !failed && work.next(p, w); ++local) {
      int tm, tn;
      tile_coords(w.tile, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
      const int m0 = tm * (2 * BM) + static_cast<int>(rank) * BM;
      const int n0 = tn * BN;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
        failed = true;
        break;
      }
      tc_fence_after();
      // A tail tile cut along K: this warp's 32 x BN slab is either parked for the
      // pair that holds piece 0, or (piece 0) completed with the parked slabs.
      const size_t my_slab = rank * 4 + quad;
      const size_t tail_base = static_cast<size_t>(w.tail) * (p.tail_split > 1 ? p.tail_split - 1 : 1);
      if (w.split > 1 && w.piece == 0) {
        int ok = 1;
        if (lane == 0)
          for (int j = 0; j < w.split - 1 && ok; ++j)
            ok = wait_flag_set(p.sk_flags + (tail_base + j) * 8 + my_slab) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
          if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
          failed = true;
          break;
        }
        __threadfence();
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + lane_base + acc * BN + c * 32, r);
        tmem_ld_wait();
        if (w.piece > 0) {
          // lane-interleaved layout: each store instruction writes 512 contiguous bytes
          float4* parked = reinterpret_cast<float4*>(
              p.sk_partials + ((tail_base + w.piece - 1) * 8 + my_slab) * (32 * BN));
#pragma unroll
          for (int j = 0; j < 8; ++j)
            parked[(c * 8 + j) * 32 + lane] =
                make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          continue;
        }
        for (int piece = 1; piece < w.split; ++piece) {
          const float4* parked = reinterpret_cast<const float4*>(
              p.sk_partials + ((tail_base + piece - 1) * 8 + my_slab) * (32 * BN));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = __ldcg(&parked[(c * 8 + j) * 32 + lane]);
            r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
            r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
            r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
            r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
          }
        }
        if (p.relu) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            r[i] = __float_as_uint(fmaxf(__uint_as_float(r[i]), p.relu_threshold));
        }
        const int col0 = n0 + c * 32;
        float* sb = stage_buf + buf * (32 * 32);
        tma_store_wait_read<1>();
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
        if (lane == 0 && col0 < p.N && m0 + quad * 32 < p.M) {
          if (p.c_evict_first)
            tma_store_2d_hint(&tmC, sb, col0, m0 + quad * 32, store_policy);
          else
            tma_store_2d(&tmC, sb, col0, m0 + quad * 32);
        }
        if (lane == 0) tma_store_commit();
        if (p.n_extra > 0 && !copiers) {
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
      }
      if (w.piece > 0) {
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicExch(p.sk_flags + (tail_base + w.piece - 1) * 8 + my_slab, 1);
      } else if (w.split > 1) {
        __syncwarp();
        if (lane == 0)  // leave the flags as the next launch expects them
          for (int j = 0; j < w.split - 1; ++j) p.sk_flags[(tail_base + j) * 8 + my_slab] = 0;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
      if (copiers && w.piece == 0 && lane == 0) {
        tma_store_wait_all<0>();  // this warp's 32 rows of the tile are in the local C
        __threadfence();
        stored[quad] = stored[quad] + 1;
      }
    }
    tma_store_wait_all<0>();
  } else if (copiers) {
    // ------------------- copier warps (broadcast to the peers) -------------------
    // Warp q copies the 32 rows that the epilogue warp of quadrant q stored, once that
    // warp has counted the tile: read from the local C (L2), 128-bit stores over NVLink.
    const int q = warp - (2 + EPI_WARPS);
    constexpr int V = BN / 4;             // float4 per tile row
    constexpr int JT = (V + 31) / 32;     // float4 per lane and row
    uint32_t seen = 0;
    PairWorkIter work(pair, num_pairs);
    PairWork w;
    while (!failed && work.next(p, w)) {
      if (w.piece != 0) continue;  // another pair stores this tile
      ++seen;
      int ok = 1;
      if (lane == 0) {
        uint64_t t0 = 0;
        for (uint32_t it = 0; stored[q] < seen; ++it) {
          if ((it & 0xff) == 0xff) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) { ok = 0; break; }
          }
        }
      }
      if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
        if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
        failed = true;
        break;
      }
      __threadfence();
      int tm, tn;
      tile_coords(w.tile, p.tiles_m, p.tiles_n, p.group_n, tm, tn);
      const int row0 = tm * (2 * BM) + static_cast<int>(rank) * BM + q * 32;
      const int n0 = tn * BN;
#pragma unroll 1
      for (int r = 0; r < 32; r += 4) {
        float4 v[4][JT];
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          const int row = row0 + r + rr;
#pragma unroll
          for (int j = 0; j < JT; ++j) {
            const int idx = j * 32 + lane;
            const int col = n0 + idx * 4;
            if (idx < V && row < p.M && col < p.N)
              v[rr][j] = __ldcg(reinterpret_cast<const float4*>(p.C + static_cast<int64_t>(row) * p.ldc + col));
          }
        }
        if (p.mc_dst != nullptr) {  // one multicast store per vector reaches every GPU
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int row = row0 + r + rr;
#pragma unroll
            for (int j = 0; j < JT; ++j) {
              const int idx = j * 32 + lane;
              const int col = n0 + idx * 4;
              if (idx < V && row < p.M && col < p.N)
                multimem_st_f4(p.mc_dst + static_cast<int64_t>(row) * p.ldc + col, v[rr][j]);
            }
          }
          continue;
        }
        for (int d = 0; d < p.n_extra; ++d) {
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int row = row0 + r + rr;
#pragma unroll
            for (int j = 0; j < JT; ++j) {
              const int idx = j * 32 + lane;
              const int col = n0 + idx * 4;
              if (idx < V && row < p.M && col < p.N)
                *reinterpret_cast<float4*>(p.extra_dst[d] + static_cast<int64_t>(row) * p.ldc + col) = v[rr][j];
            }
          }
        }
      }
    }
  }

  if (failed) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace xtc
