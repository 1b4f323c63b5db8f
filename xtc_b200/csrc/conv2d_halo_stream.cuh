// Halo-tile convolution with STREAMED weights, for layers whose filter bank does not fit in
// shared memory (3x3x128 -> 128 and deeper): stride 1, CTA pairs (conv2d_halo_pair.cuh).
//
// The im2col kernels fetch a tile's pixels once per filter tap: for a 3x3 filter 1.2 MB of
// pixels and 1.2 MB of weights go through one SM's shared memory per 128 x 128 tile of
// 256 input channels, and that fill rate, not the tensor pipe, sets their pace.  Here a pipeline
// stage is one 32-channel slab: the halo run of the tile's positions (one im2col-mode TMA copy,
// 128 + (R-1)*Wp + (S-1) pixel rows of 128 bytes, read by every tap at its own row offset) and
// the weights of ALL taps for those 32 channels and this CTA's 64 filters (two 3-D TMA copies of
// taps x 32 x 32 floats).  Two CTAs share one 256 x 128 MMA (cta_group::2): each owns 128
// consecutive positions and half of the 128 filters of the tile, so a 3x3 stage is 32 KB of
// pixels and 72 KB of weights per CTA for 36 MMAs of 256 x 128 x 8, and the tensor pipe is
// the bound again.  Work items are (position tile, filter tile) pairs; like the other halo
// kernels this one computes every position of the padded grid and stores the valid ones.
//
// Stage layout: [halo slab, rounded up to 1024 bytes][filter group 0: taps x 4 KB][group 1:
// taps x 4 KB]; a tap's block is 32 k-rows of 32 filters, the MN-major operand layout of
// conv2d_halo.cuh, and the two groups of a tap lie taps * 4096 bytes apart (the descriptor's
// leading-dimension offset).  With 16-channel slabs (SLAB = 16) everything halves: pixel rows
// of 64 bytes, tap blocks of 16 k-rows, and twice as many stages fit.
//
// Balance.  With whole work items dealt round-robin, 113 items on 74 CTA pairs are two rounds of
// which the second is half empty.  Given a workspace, the kernel deals out (work item, channel
// slab) units instead: pair p takes the contiguous range [p*U/P, (p+1)*U/P) of the U = items x
// slabs units, so a pair's first and last item may be partial.  The pair that holds an item's
// slab 0 stores it; every other pair holding some of its slabs does so at the START of its range,
// writes its raw accumulator to the workspace (per warp: [pair][CTA][warp] blocks of 32 rows,
// lane-interleaved so that every store is 512 contiguous bytes) and raises that warp's flag; the storing pair reaches that item at the END of its range, waits (bounded, normally not at
// all) for the flags of the pairs after it, adds their partials in pair order and clears the flags.
// Same bits on every run; the bits differ from the round-robin form only in where the sum over
// slabs is cut.  All pairs are resident at once (one CTA per SM, at most SMs / 2 pairs).
//
// Barriers (no multicast anywhere):
//   full[s]      leader only; both CTAs' copies of a stage report to it.
//   empty[s]     one per CTA; the leader commits to both.
//   acc_full[a]  one per CTA; the leader commits to both.
//   acc_empty[a] leader only, 8 arrivals (4 epilogue warps of each CTA).
#pragma once
#include "conv2d_halo.cuh"

namespace xtc {

constexpr int STREAM_BN = 128;

// The segments (work item, slabs [s0, s1)) of one CTA pair, in the order every role of the
// kernel walks them.
struct StreamSegments {
  bool balanced;
  int item, step, items, nslab;  // round-robin: whole items pair, pair + step, ...
  long long unit, unit_hi;       // balanced: the pair's range of (item, slab) units
  __device__ StreamSegments(const ConvHaloParams& p, int pair, int num_pairs)
      : balanced(p.sk_partials != nullptr), item(pair), step(num_pairs), items(p.tiles), nslab(p.nslab) {
    const long long units = static_cast<long long>(p.tiles) * p.nslab;
    const long long q = units / num_pairs, r = units % num_pairs;
    unit = pair * q + (pair < r ? pair : r);
    unit_hi = unit + q + (pair < r ? 1 : 0);
  }
  __device__ bool next(int& it, int& s0, int& s1) {
    if (!balanced) {
      if (item >= items) return false;
      it = item;
      s0 = 0;
      s1 = nslab;
      item += step;
      return true;
    }
    if (unit >= unit_hi) return false;
    it = static_cast<int>(unit / nslab);
    s0 = static_cast<int>(unit - static_cast<long long>(it) * nslab);
    const long long item_end = static_cast<long long>(it + 1) * nslab;
    const long long end = item_end < unit_hi ? item_end : unit_hi;
    s1 = s0 + static_cast<int>(end - unit);
    unit = end;
    return true;
  }
};
// Units of pair `pair` when `units` are dealt out evenly to `num_pairs` pairs.
__device__ __forceinline__ long long stream_units_of(long long units, int num_pairs, int pair) {
  return units / num_pairs + (pair < units % num_pairs ? 1 : 0);
}

template <bool DUAL, int SLAB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(HALO_THREADS, 1)
conv2d_halo_stream_kernel(const __grid_constant__ CUtensorMap tmX,
                          const __grid_constant__ CUtensorMap tmW, const ConvHaloParams p) {
  using namespace dev;
  static_assert(SLAB == 16 || SLAB == 32, "slabs are 16 or 32 channels wide");
  constexpr int BN = STREAM_BN;
  constexpr int HALF = BN / 2;
  constexpr int ROW = SLAB * 4;                   // bytes per pixel row of a stage
  constexpr uint32_t TAP_BLOCK = SLAB * 128;      // one tap's weights for 32 filters: SLAB k rows of 128 B
  constexpr int NACC = DUAL ? 2 : 1;  // accumulators per tile, one per issuing thread
  constexpr uint32_t TMEM_COLS = 2 * NACC * BN;
  static_assert(TMEM_COLS <= 512, "accumulators do not fit in TMEM");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* ring = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(p.stages) * p.stage_bytes);
  uint64_t* full = bars;           // [stages]
  uint64_t* empty = bars + 8;      // [stages]
  uint64_t* acc_full = bars + 16;  // [2]
  uint64_t* acc_empty = bars + 18; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NACC);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], NACC);
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
  cluster_sync_all();
  tc_fence_after();
  grid_dependency_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int plane = p.Hp * p.Wp;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  bool failed = false;

  if (warp == 0) {
    // ------------------------------ producer --------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t group_bytes = static_cast<uint32_t>(p.taps) * TAP_BLOCK;
      StreamSegments segs(p, pair, num_pairs);
      int tile, s0, s1;
      while (!failed && segs.next(tile, s0, s1)) {
        const int ptile = tile / p.ntiles_n;
        const int ntile = tile - ptile * p.ntiles_n;
        long long q0 = static_cast<long long>(ptile) * (2 * BM) + static_cast<long long>(rank) * BM;
        if (q0 >= p.Q) q0 = 0;  // nothing of this half is stored; fetch something valid
        const int img = static_cast<int>(q0 / plane);
        const int rem = static_cast<int>(q0 - static_cast<long long>(img) * plane);
        const int ih = rem / p.Wp - p.pad_top;
        const int iw = rem % p.Wp - p.pad_left;
        const int f0 = ntile * BN + static_cast<int>(rank) * HALF;
        for (int slab = s0; slab < s1; ++slab) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_EMPTY);
            failed = true;
            break;
          }
          if (leader)
            mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(2 * (p.stage_tx + p.wts_tx)));
          uint8_t* dst = ring + static_cast<size_t>(stage) * p.stage_bytes;
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          tma_load_im2col_4d_pair(dst, &tmX, bar, slab * SLAB, iw, ih, img, 0, 0);
#pragma unroll
          for (int g = 0; g < HALF / 32; ++g)
            tma_load_3d_pair(dst + p.wts_offset + g * group_bytes, &tmW, bar, f0 + g * 32, slab * SLAB, 0);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp <= 2) {
    // ------------------------ MMA issuers (leader CTA) ------------------------
    // Warps 1 and 2 share the taps of every slab (see conv2d_halo.cuh on why two).
    const int w = warp - 1;
    if (lane == 0 && leader && w < NACC) {
      constexpr uint32_t idesc = umma_idesc_tf32(2 * BM, BN, false, true);
      const int t0 = DUAL ? (w == 0 ? 0 : (p.taps + 1) / 2) : 0;
      const int t1 = DUAL ? (w == 0 ? (p.taps + 1) / 2 : p.taps) : p.taps;
      const int r0 = t0 / p.S, tap_s0 = t0 - r0 * p.S;
      // A: K-major rows of ROW bytes, 8-row swizzle atoms
      const uint32_t a_hi = umma_desc_hi(8 * ROW, static_cast<uint32_t>(SLAB == 32 ? UMMA_SWIZZLE_128B
                                                                                  : UMMA_SWIZZLE_64B));
      const uint32_t b_hi = umma_desc_hi(512, static_cast<uint32_t>(UMMA_SWIZZLE_128B_BASE32B));
      const uint32_t group_bytes = static_cast<uint32_t>(p.taps) * TAP_BLOCK;
      constexpr uint32_t PIX = ROW >> 4;                              // one pixel row, >> 4
      const uint32_t row_step = static_cast<uint32_t>(p.Wp) * PIX;  // one image row down
      const uint32_t a_first = static_cast<uint32_t>(r0) * row_step;
      int stage = 0;
      uint32_t phase = 0;
      StreamSegments segs(p, pair, num_pairs);
      int tile, s0, s1;
      for (int local = 0; !failed && segs.next(tile, s0, s1); ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_DRAIN);
          failed = true;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (acc * NACC + w) * BN;
        for (int slab = s0; slab < s1; ++slab) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(ring + static_cast<size_t>(stage) * p.stage_bytes);
          uint32_t a_row = umma_desc_lo(sA, 16) + a_first;
          uint32_t b_lo = umma_desc_lo(sA + static_cast<uint32_t>(p.wts_offset) +
                                           static_cast<uint32_t>(t0) * TAP_BLOCK, group_bytes);
          uint32_t first = slab == s0 ? 0u : 1u;  // a segment's first MMA overwrites its accumulator
          for (int tap = t0, s = tap_s0; tap < t1; ++tap) {
            const uint32_t a_lo = a_row + static_cast<uint32_t>(s) * PIX;
#pragma unroll
            for (int kk = 0; kk < SLAB / 8; ++kk) {
              umma_tf32_pair(d_tmem, umma_desc_pack(a_lo + kk * 2, a_hi),
                             umma_desc_pack(b_lo + kk * 64, b_hi), idesc, first | (kk != 0));
            }
            first = 1u;
            b_lo += TAP_BLOCK >> 4;
            if (++s == p.S) {
              s = 0;
              a_row += row_step;
            }
          }
          const uint32_t e = smem_u32(&empty[stage]);
          tc_commit_pair(map_to_cta(e, 0));
          tc_commit_pair(map_to_cta(e, 1));
          if (++stage == p.stages) {
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
  } else {
    // --------------------------- epilogue (both CTAs) --------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const bool vec_ok = (p.F % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0);
    const bool wide_ok = (p.F % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 31) == 0);
    // balanced form: the rows of this warp travel on their own (partials and flags per
    // (pair, CTA, warp)), so no warp waits for another one of its CTA
    const int my_slab = static_cast<int>(rank) * EPI_WARPS + quad;
    const long long units = static_cast<long long>(p.tiles) * p.nslab;
    constexpr int SLAB_FLOATS = 32 * BN;  // 32 rows x BN columns of one warp
    StreamSegments segs(p, pair, num_pairs);
    int tile, s0, s1;
    for (int local = 0; !failed && segs.next(tile, s0, s1); ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
        failed = true;
        break;
      }
      tc_fence_after();
      const bool stores = s0 == 0;  // this pair holds the item's first slab: it writes the output
      // the pairs after this one that hold the rest of the item's slabs
      int helpers = 0;
      if (stores && s1 < p.nslab) {
        long long rest = p.nslab - s1;
        for (int h = pair + 1; rest > 0 && h < num_pairs; ++h, ++helpers)
          rest -= stream_units_of(units, num_pairs, h);
        int ok = 1;
        if (lane == 0)
          for (int h = 1; h <= helpers && ok; ++h)
            ok = wait_flag_set(p.sk_flags + (pair + h) * (2 * EPI_WARPS) + my_slab) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, ok, 0) == 0) {
          if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
          failed = true;
          break;
        }
        __threadfence();
      }
      const int ptile = tile / p.ntiles_n;
      const int n0 = (tile - ptile * p.ntiles_n) * BN;
      const long long q = static_cast<long long>(ptile) * (2 * BM) + static_cast<long long>(rank) * BM +
                          quad * 32 + lane;
      const int img = static_cast<int>(q / plane);
      const int rem = static_cast<int>(q - static_cast<long long>(img) * plane);
      const int oh = rem / p.Wp;
      const int ow = rem - oh * p.Wp;
      const bool valid = q < p.Q && oh < p.OH && ow < p.OW;
      float* dst = p.Y + ((static_cast<long long>(img) * p.OH + oh) * p.OW + ow) * p.F + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + lane_base + acc * NACC * BN + c * 32, r);
        if (DUAL) {
          uint32_t r2[32];
          tmem_ld_32x32(tmem_base + lane_base + (acc * NACC + 1) * BN + c * 32, r2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
        } else {
          tmem_ld_wait();
        }
        if (!stores) {
          // a later part of an item: the raw sums go to the pair that stores it
          // (lane-interleaved: each store instruction writes 512 contiguous bytes)
          float4* parked = reinterpret_cast<float4*>(
              p.sk_partials + (static_cast<size_t>(pair) * (2 * EPI_WARPS) + my_slab) * SLAB_FLOATS);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            parked[(c * 8 + j) * 32 + lane] =
                make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          continue;
        }
        for (int h = 1; h <= helpers; ++h) {  // pair order: the same bits on every run
          const float4* parked = reinterpret_cast<const float4*>(
              p.sk_partials + (static_cast<size_t>(pair + h) * (2 * EPI_WARPS) + my_slab) * SLAB_FLOATS);
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
        if (valid) {
          const int col0 = c * 32;
          if (wide_ok && n0 + col0 + 32 <= p.F) {
#pragma unroll
            for (int j = 0; j < 4; ++j) st_global_f8(dst + col0 + 8 * j, r + 8 * j);
          } else if (vec_ok && n0 + col0 + 32 <= p.F) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<float4*>(dst + col0)[j] =
                  make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                              __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + col0 + i < p.F) dst[col0 + i] = __uint_as_float(r[i]);
          }
        }
      }
      if (!stores) {  // publish the partial
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicExch(p.sk_flags + pair * (2 * EPI_WARPS) + my_slab, 1);
      } else if (helpers > 0) {
        __syncwarp();  // every lane has read the partials
        if (lane == 0)  // leave the flags as the next launch expects them
          for (int h = 1; h <= helpers; ++h) p.sk_flags[(pair + h) * (2 * EPI_WARPS) + my_slab] = 0;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
    }
  }

  if (failed) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace xtc
