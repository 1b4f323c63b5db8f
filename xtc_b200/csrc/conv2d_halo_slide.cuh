// Resident-weights convolution (conv2d_halo.cuh) with a sliding input window.
//
// conv2d_halo.cuh gives a CTA every (number of CTAs)-th tile of 128 output positions and fetches
// the whole halo run of a tile, 128 + (R-1)*Wp + (S-1) positions, per 32-channel slab: 246
// positions for 128 outputs on a 3x3 filter over 58-wide rows, and with the filter bank taking
// 147 KB only two such runs fit, so a run is fetched while nothing but the other one is being
// multiplied and its latency shows (a tile takes 4.7k clocks where its MMAs need 4.1k).
//
// Here a CTA takes a RUN of consecutive tiles, so that the halo of a tile is the first part of the
// next tile's input, and the input streams through a ring of 128-position chunks: tile i of a run
// reads chunks i and i+1 (P <= 256 positions), each chunk is fetched once per slab (one
// im2col-mode TMA copy of 16 KB), and three chunks beyond the one being read can be in flight.
// The ring has four slots plus a fifth that mirrors slot 0, so that the tile whose first chunk
// sits in slot 3 finds its second chunk right behind it (an MMA operand must be contiguous).
//
// Streaming the positions of a whole run means going through the run once per slab, so the
// accumulators of all tiles of the run live in TMEM at once (256 / BN tiles; longer runs are
// processed in groups): pass 0 multiplies channel slab 0 of every tile, pass 1 adds slab 1, ...
// Two threads issue MMAs, each half of the taps of every tile into an accumulator of its own
// (one thread alone issues an MMA per 57 clocks, two reach the 48 the shared-memory feed
// allows; the result does not depend on how the two streams interleave); two sets of four
// epilogue warps add the two accumulators of a tile and store it as the last pass completes it.
// (Giving the two threads alternate tiles instead keeps two windows in use at once, for which
// four slots are too few: 23.9 us on the 3x3x64 -> 64 layer.)
//
// Barriers: full[4] (a chunk and, where it has one, its mirror copy have landed), empty[4] (four
// arrivals: the two tiles that read a chunk, two issuing threads each; the first and last chunk
// of a pass are read by one tile, whose threads arrive twice), acc_full[4] (two arrivals) /
// acc_empty[4] per tile of a group, wbar (filter bank).
#pragma once
#include "conv2d_halo.cuh"

namespace xtc {

constexpr int SLIDE_CHUNK = 128;                    // positions per chunk = positions per tile
constexpr int SLIDE_SLOT_BYTES = SLIDE_CHUNK * 128;  // 32 channels x 4 bytes per position
constexpr int SLIDE_SLOTS = 4;                       // + 1 mirror of slot 0
constexpr int SLIDE_THREADS = (3 + 8) * 32;          // producer, two issuers, two epilogue sets

template <int BN>
__global__ void __launch_bounds__(SLIDE_THREADS, 1)
conv2d_halo_slide_kernel(const __grid_constant__ CUtensorMap tmX,
                         const __grid_constant__ CUtensorMap tmW, const ConvHaloParams p) {
  using namespace dev;
  constexpr int GT = 256 / BN;      // tiles per group: two accumulators each
  constexpr int WBLOCK = BN * 128;  // bytes of weights per (tap, 32-channel block)
  static_assert(BN == 64 || BN == 128, "64 or 128 filters per tile");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* wts = smem;
  uint8_t* ring = wts + static_cast<size_t>(p.taps) * p.nblk * WBLOCK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (SLIDE_SLOTS + 1) * SLIDE_SLOT_BYTES);
  uint64_t* full = bars;            // [4]
  uint64_t* empty = bars + 4;       // [4]
  uint64_t* acc_full = bars + 8;    // [8]
  uint64_t* acc_empty = bars + 16;  // [8]
  uint64_t* wbar = bars + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
    for (int s = 0; s < SLIDE_SLOTS; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 4);
    }
    for (int a = 0; a < 8; ++a) {
      mbar_init(&acc_full[a], 2);
      mbar_init(&acc_empty[a], EPI_WARPS);
    }
    mbar_init(wbar, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dependency_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int plane = p.Hp * p.Wp;
  // this CTA's run of consecutive tiles
  const int base = p.tiles / static_cast<int>(gridDim.x);
  const int extra = p.tiles - base * static_cast<int>(gridDim.x);
  const int bid = static_cast<int>(blockIdx.x);
  const int n = base + (bid < extra ? 1 : 0);
  const int T0 = bid * base + (bid < extra ? bid : extra);
  bool failed = false;

  if (warp == 0) {
    // ------------------------------ producer --------------------------------
    auto issue_chunk = [&](int tile, int slab, int g, bool mirror) {
      const long long q0 = static_cast<long long>(tile) * SLIDE_CHUNK;
      const int img = static_cast<int>(q0 / plane);
      const int rem = static_cast<int>(q0 - static_cast<long long>(img) * plane);
      const int ih = rem / p.Wp - p.pad_top;
      const int iw = rem % p.Wp - p.pad_left;
      const int s = g & 3;
      if (tile >= p.tiles) {
        // the chunk behind the last tile of the grid: it only feeds output positions that do
        // not exist, so nothing is fetched and the barrier is completed by hand
        mbar_arrive(&full[s]);
        return;
      }
      mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(mirror ? 2 * SLIDE_SLOT_BYTES : SLIDE_SLOT_BYTES));
      tma_load_im2col_4d(ring + s * SLIDE_SLOT_BYTES, &tmX, &full[s], slab * 32, iw, ih, img, 0, 0);
      if (mirror)
        tma_load_im2col_4d(ring + SLIDE_SLOTS * SLIDE_SLOT_BYTES, &tmX, &full[s], slab * 32, iw, ih, img,
                           0, 0);
    };
    // the first tile's two chunks (from DRAM) before the filter bank (from L2), the next two
    // after it; all slots are free
    const int m0 = n < GT ? n : GT;
    const int pre = m0 + 1 < SLIDE_SLOTS ? m0 + 1 : SLIDE_SLOTS;
    if (lane == 0) {
      for (int j = 0; j < 2 && j < pre; ++j) issue_chunk(T0 + j, 0, j, false);
      mbar_arrive_expect_tx(wbar, static_cast<uint32_t>(p.taps * p.nblk * WBLOCK));
    }
    __syncwarp();
    {
      const int copies = p.taps * p.nblk * (BN / 32);
      for (int i = lane; i < copies; i += 32) {
        const int g = i % (BN / 32);
        const int tb = i / (BN / 32);  // tap * nblk + blk
        const int tap = tb / p.nblk, blk = tb - tap * p.nblk;
        tma_load_2d(wts + static_cast<size_t>(tb) * WBLOCK + g * 4096, &tmW, wbar, g * 32,
                    tap * p.C + blk * 32);
      }
    }
    if (lane == 0) {
      for (int j = 2; j < pre; ++j) issue_chunk(T0 + j, 0, j, false);
      XTC_TRACE_DECL(0);
      XTC_TRACE_MARK();  // bank and first chunks issued
      int g0 = 0;
      for (int gs = 0; gs < n && !failed; gs += GT) {
        const int m = n - gs < GT ? n - gs : GT;
        for (int pass = 0; pass < p.nslab && !failed; ++pass) {
          for (int j = 0; j <= m; ++j) {
            const int g = g0 + j;
            if (g < pre) continue;  // already out
            if (g >= SLIDE_SLOTS && !mbar_wait(&empty[g & 3], ((g >> 2) - 1) & 1)) {
              atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_EMPTY);
              failed = true;
              break;
            }
            XTC_TRACE_MARK();  // slot free: chunk issued
            issue_chunk(T0 + gs + j, pass, g, (g & 3) == 0 && j > 0);
          }
          g0 += m + 1;
        }
      }
    }
  } else if (warp <= 2) {
    // ------------------------------ MMA issuers ------------------------------
    const int w = warp - 1;
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_tf32(BM, BN, false, true);
      XTC_TRACE_DECL(1 + w);
      XTC_TRACE_MARK();  // start
      if (!mbar_wait(wbar, 0)) {
        atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
        failed = true;
      }
      XTC_TRACE_MARK();  // bank landed
      // this thread's share of the taps
      const int t0 = w == 0 ? 0 : (p.taps + 1) / 2;
      const int t1 = w == 0 ? (p.taps + 1) / 2 : p.taps;
      const int r0 = t0 / p.S, s0 = t0 - r0 * p.S;
      const uint32_t w0 = smem_u32(wts) + static_cast<uint32_t>(t0) * p.nblk * WBLOCK;
      const uint32_t a_hi = umma_desc_hi(8 * 128, static_cast<uint32_t>(UMMA_SWIZZLE_128B));
      const uint32_t b_hi = umma_desc_hi(512, static_cast<uint32_t>(UMMA_SWIZZLE_128B_BASE32B));
      const uint32_t b_step = static_cast<uint32_t>(p.nblk) * (WBLOCK >> 4);
      constexpr uint32_t PIX = 128 >> 4;                            // one position, >> 4
      const uint32_t row_step = static_cast<uint32_t>(p.Wp) * PIX;  // one image row down
      const uint32_t a_first = static_cast<uint32_t>(r0) * row_step;
      int g0 = 0, grp = 0;
      for (int gs = 0; gs < n && !failed; gs += GT, ++grp) {
        const int m = n - gs < GT ? n - gs : GT;
        for (int pass = 0; pass < p.nslab && !failed; ++pass) {
          for (int a = 0; a < m; ++a) {
            if (pass == 0 && grp > 0 && !mbar_wait(&acc_empty[a], (grp - 1) & 1)) {
              atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_DRAIN);
              failed = true;
              break;
            }
            const int G = g0 + a;
            if (!mbar_wait(&full[G & 3], (G >> 2) & 1) ||
                !mbar_wait(&full[(G + 1) & 3], ((G + 1) >> 2) & 1)) {
              atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
              failed = true;
              break;
            }
            tc_fence_after();
            XTC_TRACE_MARK();  // window landed
            const uint32_t d_tmem = tmem_base + (a * 2 + w) * BN;
            // slot 3 is followed by the mirror of slot 0: the window is contiguous either way
            uint32_t a_row = umma_desc_lo(smem_u32(ring + (G & 3) * SLIDE_SLOT_BYTES), 16) + a_first;
            uint32_t b_lo = umma_desc_lo(w0 + static_cast<uint32_t>(pass) * WBLOCK, 4096);
            uint32_t first = pass == 0 ? 0u : 1u;
            for (int tap = t0, s = s0; tap < t1; ++tap) {
              const uint32_t a_lo = a_row + static_cast<uint32_t>(s) * PIX;
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                umma_tf32(d_tmem, umma_desc_pack(a_lo + kk * 2, a_hi),
                          umma_desc_pack(b_lo + kk * 64, b_hi), idesc, first | (kk != 0));
              }
              first = 1u;
              b_lo += b_step;
              if (++s == p.S) {
                s = 0;
                a_row += row_step;
              }
            }
            // a chunk is released by four arrivals: two tiles, two threads each; the first chunk
            // of a pass and the last are read by one tile only, whose threads arrive for both
            tc_commit(&empty[G & 3]);
            if (a == 0) tc_commit(&empty[G & 3]);
            tc_commit(&empty[(G + 1) & 3]);
            if (a == m - 1) tc_commit(&empty[(G + 1) & 3]);
            if (pass == p.nslab - 1) tc_commit(&acc_full[a]);
            XTC_TRACE_MARK();  // tile-slab issued
          }
          g0 += m + 1;
        }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3;         // TMEM lanes 32 * (warp % 4) ...
    const int set = (warp - 3) >> 2;   // the even or the odd tiles of a group
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const bool vec_ok = (p.F % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0);
    const bool wide_ok = (p.F % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 31) == 0);
    XTC_TRACE_DECL(3);
#ifdef XTC_TRACE
    if (quad != 0 || lane != 0 || set != 0) _tb = nullptr;
#endif
    int grp = 0;
    for (int gs = 0; gs < n && !failed; gs += GT, ++grp) {
      const int m = n - gs < GT ? n - gs : GT;
      for (int a = set; a < m; a += 2) {
        if (!mbar_wait(&acc_full[a], grp & 1)) {
          if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
          failed = true;
          break;
        }
        tc_fence_after();
        XTC_TRACE_MARK();  // accumulators ready
        const long long q = static_cast<long long>(T0 + gs + a) * BM + quad * 32 + lane;
        const int img = static_cast<int>(q / plane);
        const int rem = static_cast<int>(q - static_cast<long long>(img) * plane);
        const int oh = rem / p.Wp;
        const int ow = rem - oh * p.Wp;
        const bool valid = q < p.Q && oh < p.OH && ow < p.OW;
        float* dst = p.Y + ((static_cast<long long>(img) * p.OH + oh) * p.OW + ow) * p.F;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32], r2[32];
          tmem_ld_32x32(tmem_base + lane_base + (a * 2) * BN + c * 32, r);
          tmem_ld_32x32(tmem_base + lane_base + (a * 2 + 1) * BN + c * 32, r2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
          if (p.relu) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              r[i] = __float_as_uint(fmaxf(__uint_as_float(r[i]), p.relu_threshold));
          }
          if (valid) {
            const int col0 = c * 32;
            if (wide_ok && col0 + 32 <= p.F) {
#pragma unroll
              for (int j = 0; j < 4; ++j) st_global_f8(dst + col0 + 8 * j, r + 8 * j);
            } else if (vec_ok && col0 + 32 <= p.F) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                reinterpret_cast<float4*>(dst + col0)[j] =
                    make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.F) dst[col0 + i] = __uint_as_float(r[i]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        XTC_TRACE_MARK();  // tile stored
        if (lane == 0) mbar_arrive(&acc_empty[a]);
      }
    }
  }

  if (failed) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  // the weights copy must have landed before this CTA's shared memory is released
  if (warp == 0 && lane == 0 && !failed) mbar_wait(wbar, 0);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace xtc
