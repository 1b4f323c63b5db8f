// Resident-weights / halo-tile convolution (conv2d_halo.cuh) with two filter taps per MMA.
//
// With at most 64 filters a 128 x 64 x 8 MMA is bound by its shared-memory reads: 4 KB of
// pixels for 2 KB of weights, 48 clocks for 32 clocks of arithmetic.  This kernel halves the
// pixel reads.  Two taps that are neighbours along the filter row, (r, s) and (r, s+1), read
// pixel runs that differ by exactly one position, so ONE pixel operand can serve both if the
// second tap's result is allowed to land one row lower:
//
//   A = pixels q + r*Wp + s        (128 rows of the halo run, as in conv2d_halo.cuh)
//   B = [ W[r,s] | W[r,s+1] ]      (N = 128: the two taps' filters side by side)
//   D[m][0:64]   += tap (r,s)   for output position q0 + m
//   D[m][64:128] += tap (r,s+1) for output position q0 + m - 1
//
// and the epilogue forms  out[q0+m] = D[m][0:64] + D[m+1][64:128]  with one register
// shuffle per value (row m+1 is the next lane; the four rows that cross a warp boundary go
// through 1 KB of shared memory).  A filter row of odd length leaves one single tap, issued
// as a 128 x 64 x 8 MMA.  For a 3x3 filter a K step of 8 is then 3 MMAs of 128x128x8
// (8 KB of reads, 64 clocks, arithmetic 64) and 3 of 128x64x8 (48 clocks) instead of 9 of
// 128x64x8: 336 clocks instead of 432, in 6 instructions instead of 9.
//
// Tiles advance by 127 positions (row 127 of a tile has no row below it).  Two issuing
// threads as in conv2d_halo.cuh, but split by kind: warp 1 issues the paired MMAs into
// accumulator A (128 columns), warp 2 the single taps into accumulator B (64 columns); the
// epilogue adds the two, so the result does not depend on how the streams interleave.
// Both accumulators are double buffered: 2 x (128 + 64) = 384 of 512 TMEM columns.
//
// Measured on 32x56x56x64 -> 64, 3x3 (B200): the MMA phases do run 1.5 times faster than in
// conv2d_halo.cuh (5.5 us per 32 channels against 8.4 us), but the heavier epilogue (three
// accumulator reads, the row exchange) then sets the pace: 24.9 us per call against 22.8 us.
// The library therefore only uses this kernel when it is asked for (variant = 3).
//
// Filter bank layout: [r][32-channel block][s][32-filter group] blocks of 32 k-rows x 128 B,
// so that the groups of taps s and s+1 follow each other at the 4096-byte pitch an MN-major
// operand of 128 columns needs.
#pragma once
#include "conv2d_halo.cuh"

namespace xtc {

constexpr int TAPS_TILE = BM - 1;  // output positions a tile produces

template <int SLAB>
__global__ void __launch_bounds__(HALO_THREADS, 1)
conv2d_halo_taps_kernel(const __grid_constant__ CUtensorMap tmX,
                        const __grid_constant__ CUtensorMap tmW, const ConvHaloParams p) {
  using namespace dev;
  constexpr int BN = 64;
  constexpr int ACC_COLS = 3 * BN;  // accumulator A: 128 columns, accumulator B: 64
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(SLAB == 16 || SLAB == 32, "slabs are 16 or 32 channels wide");
  constexpr int ROW = SLAB * 4;     // bytes per pixel row of a stage
  constexpr int WBLOCK = BN * 128;  // bytes of one tap's weights per 32-channel block

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* wts = smem;
  uint8_t* ring = wts + static_cast<size_t>(p.taps) * p.nblk * WBLOCK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(p.stages) * p.stage_bytes);
  uint64_t* full = bars;           // [stages]
  uint64_t* empty = bars + 8;      // [stages]
  uint64_t* acc_full = bars + 16;  // [2]
  uint64_t* acc_empty = bars + 18; // [2]
  uint64_t* wbar = bars + 20;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  // rows that cross a warp boundary: [tile parity][column chunk][warp 1..3][32 floats]
  float* xch = reinterpret_cast<float*>(bars + 32);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int R = p.taps / p.S;
  const int pairs = p.S / 2;          // tap pairs per filter row
  const bool single = (p.S & 1) != 0; // a last tap without partner
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 2);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 2);
      mbar_init(&acc_empty[a], EPI_WARPS);
    }
    mbar_init(wbar, 1);
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
  const int plane = p.Hp * p.Wp;
  bool failed = false;

  if (warp == 0) {
    // ------------------------------ producer --------------------------------
    // The filter bank, once: one thread announces the bytes, then every lane issues its share
    // of the copies.  Block (r, blk, s, g) holds k rows [blk*32, +32) of tap (r, s), filters
    // [g*32, +32).
    if (lane == 0) mbar_arrive_expect_tx(wbar, static_cast<uint32_t>(p.taps * p.nblk * WBLOCK));
    __syncwarp();
    {
      const int copies = p.taps * p.nblk * (BN / 32);
      for (int i = lane; i < copies; i += 32) {
        const int g = i % (BN / 32);
        int rest = i / (BN / 32);  // (r * nblk + blk) * S + s
        const int s = rest % p.S;
        rest /= p.S;
        const int blk = rest % p.nblk, r = rest / p.nblk;
        tma_load_2d(wts + static_cast<size_t>(i) * 4096, &tmW, wbar, g * 32,
                    (r * p.S + s) * p.C + blk * 32);
      }
    }
    if (lane == 0) {
      XTC_TRACE_DECL(0);
      XTC_TRACE_MARK();  // start
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < p.tiles && !failed; tile += gridDim.x) {
        const long long q0 = static_cast<long long>(tile) * TAPS_TILE;
        const int img = static_cast<int>(q0 / plane);
        const int rem = static_cast<int>(q0 - static_cast<long long>(img) * plane);
        const int ih = rem / p.Wp - p.pad_top;
        const int iw = rem % p.Wp - p.pad_left;
        for (int slab = 0; slab < p.nslab; ++slab) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_EMPTY);
            failed = true;
            break;
          }
          XTC_TRACE_MARK();  // stage free: load issued
          mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(p.stage_tx));
          tma_load_im2col_4d(ring + static_cast<size_t>(stage) * p.stage_bytes, &tmX, &full[stage],
                             slab * SLAB, iw, ih, img, 0, 0);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp <= 2) {
    // ------------------------------ MMA issuers ------------------------------
    // w = 0: the tap pairs, N = 128, into accumulator A; w = 1: the single taps, N = 64,
    // into accumulator B.  Both walk the same stages and arrive on the same barriers.
    const int w = warp - 1;
    if (lane == 0) {
      constexpr uint32_t idesc_pair = umma_idesc_tf32(BM, 2 * BN, false, true);
      constexpr uint32_t idesc_one = umma_idesc_tf32(BM, BN, false, true);
      XTC_TRACE_DECL(1 + w);
      XTC_TRACE_MARK();  // start
      if (!mbar_wait(wbar, 0)) {
        atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
        failed = true;
      }
      XTC_TRACE_MARK();  // bank landed
      const uint32_t a_hi = umma_desc_hi(8 * ROW, static_cast<uint32_t>(SLAB == 32 ? UMMA_SWIZZLE_128B
                                                                                  : UMMA_SWIZZLE_64B));
      const uint32_t b_hi = umma_desc_hi(512, static_cast<uint32_t>(UMMA_SWIZZLE_128B_BASE32B));
      constexpr uint32_t PIX = ROW >> 4;                            // one pixel row, >> 4
      const uint32_t row_step = static_cast<uint32_t>(p.Wp) * PIX;  // one image row down
      const uint32_t r_step = static_cast<uint32_t>(p.nblk) * p.S * (WBLOCK >> 4);  // next filter row
      const int n_mine = w == 0 ? pairs : (single ? 1 : 0);  // MMAs per filter row and K step
      const uint32_t s_first = w == 0 ? 0u : static_cast<uint32_t>(p.S - 1);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      for (int tile = blockIdx.x; tile < p.tiles && !failed; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_DRAIN);
          failed = true;
          break;
        }
        tc_fence_after();
        XTC_TRACE_MARK();  // accumulator free
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS + (w == 0 ? 0 : 2 * BN);
        for (int slab = 0; slab < p.nslab; ++slab) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
            failed = true;
            break;
          }
          XTC_TRACE_MARK();  // slab landed
          const uint32_t sA = smem_u32(ring + static_cast<size_t>(stage) * p.stage_bytes);
          // pixel run at filter column s_first; k rows [slab*SLAB, +SLAB) of that tap's block
          uint32_t a_row = umma_desc_lo(sA, 16) + s_first * PIX;
          const uint32_t k0 = static_cast<uint32_t>(slab) * SLAB;
          uint32_t b_row = umma_desc_lo(smem_u32(wts) + ((k0 >> 5) * p.S + s_first) * WBLOCK +
                                            (k0 & 31u) * 128u, 4096);
          uint32_t first = slab == 0 ? 0u : 1u;
          for (int r = 0; r < R; ++r) {
            uint32_t a_lo = a_row, b_lo = b_row;
            for (int j = 0; j < n_mine; ++j) {
#pragma unroll
              for (int kk = 0; kk < SLAB / 8; ++kk)
                umma_tf32(d_tmem, umma_desc_pack(a_lo + kk * 2, a_hi),
                          umma_desc_pack(b_lo + kk * 64, b_hi), w == 0 ? idesc_pair : idesc_one,
                          first | (kk != 0));
              first = 1u;
              a_lo += 2 * PIX;               // the next pair starts two filter columns on
              b_lo += 2 * (WBLOCK >> 4);
            }
            a_row += row_step;
            b_row += r_step;
          }
          tc_commit(&empty[stage]);
          XTC_TRACE_MARK();  // slab issued
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!failed) tc_commit(&acc_full[acc]);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const bool vec_ok = (p.F % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0);
    const bool wide_ok = (p.F % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 31) == 0);
    const int m = quad * 32 + lane;  // row of the tile = output position q0 + m
    XTC_TRACE_DECL(3);
    if (quad != 0 || lane != 0) {
#ifdef XTC_TRACE
      _tb = nullptr;
#endif
    }
    int local = 0;
    for (int tile = blockIdx.x; tile < p.tiles && !failed; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase)) {
        if (lane == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_ACC);
        failed = true;
        break;
      }
      tc_fence_after();
      XTC_TRACE_MARK();  // accumulator ready
      const long long q = static_cast<long long>(tile) * TAPS_TILE + m;
      const int img = static_cast<int>(q / plane);
      const int rem = static_cast<int>(q - static_cast<long long>(img) * plane);
      const int oh = rem / p.Wp;
      const int ow = rem - oh * p.Wp;
      const bool valid = m < TAPS_TILE && q < p.Q && oh < p.OH && ow < p.OW;
      float* dst = p.Y + ((static_cast<long long>(img) * p.OH + oh) * p.OW + ow) * p.F;
      const uint32_t t0 = tmem_base + lane_base + acc * ACC_COLS;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t lo[32], up[32];
        tmem_ld_32x32(t0 + c * 32, lo);           // this row, first tap of the pairs
        tmem_ld_32x32(t0 + BN + c * 32, up);      // this row, second tap: belongs one row up
        tmem_ld_wait();
        // the row below lives in the next lane; across a warp boundary, in shared memory
        float* slot = xch + (((local & 1) * 2 + c) * 3) * 32;
        if (lane == 0 && quad > 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) slot[(quad - 1) * 32 + i] = __uint_as_float(up[i]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float below = __shfl_down_sync(0xffffffffu, __uint_as_float(up[i]), 1);
          if (lane == 31 && quad < 3) below = slot[quad * 32 + i];
          lo[i] = __float_as_uint(__uint_as_float(lo[i]) + below);
        }
        if (single) {
          tmem_ld_32x32(t0 + 2 * BN + c * 32, up);  // the unpaired tap, this row
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            lo[i] = __float_as_uint(__uint_as_float(lo[i]) + __uint_as_float(up[i]));
        }
        if (p.relu) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            lo[i] = __float_as_uint(fmaxf(__uint_as_float(lo[i]), p.relu_threshold));
        }
        // (Transposing the block across the warp so that each store writes one whole 128-byte
        // line was measured slower: 26.1 us against 24.9 us on 32x56x56x64 -> 64.)
        if (valid) {
          const int col0 = c * 32;
          if (wide_ok && col0 + 32 <= p.F) {
#pragma unroll
            for (int j = 0; j < 4; ++j) st_global_f8(dst + col0 + 8 * j, lo + 8 * j);
          } else if (vec_ok && col0 + 32 <= p.F) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<float4*>(dst + col0)[j] =
                  make_float4(__uint_as_float(lo[4 * j]), __uint_as_float(lo[4 * j + 1]),
                              __uint_as_float(lo[4 * j + 2]), __uint_as_float(lo[4 * j + 3]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col0 + i < p.F) dst[col0 + i] = __uint_as_float(lo[i]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      XTC_TRACE_MARK();  // tile stored
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace xtc
