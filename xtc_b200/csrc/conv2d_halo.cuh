// Stride-1 NHWC convolution with resident weights and halo tiles.
//
// The im2col kernel fetches every input pixel once per filter tap (R*S times)
// and every weight once per output tile; both come from L2 and the fill rate
// of shared memory is what bounds it.  This kernel removes both re-fetches:
//
//  * the whole filter bank [R*S*C, F] is loaded into shared memory once per CTA
//    and stays there (it must fit: R*S*C*BN*4 bytes);
//  * output positions are numbered over the PADDED image grid,
//      q = (b*Hp + oh)*Wp + ow,   Hp = H + pads, Wp = W + pads,
//    so that the input pixel tap (r, s) needs for position q is simply pixel
//    q + r*Wp + s of the zero-padded input in the same numbering.  A tile of
//    128 consecutive positions therefore needs ONE run of
//    P = 128 + (R-1)*Wp + (S-1) consecutive padded pixels, fetched once per
//    32-channel slab by a single im2col-mode TMA copy whose bounding box is the
//    padded image (out-of-bounds pixels, i.e. the padding, arrive as zeros);
//  * the MMA of tap (r, s) reads its A operand from that run at a byte offset of
//    (r*Wp + s)*128: a K-major SWIZZLE_128B operand may start at any 128-byte
//    row because the swizzle is a function of the absolute shared-memory address.
//
// Positions with oh >= OH or ow >= OW are computed and not stored (a few
// percent of extra MMA work).  Accumulators are double buffered in TMEM; relu is
// fused into the epilogue.
//
// Slab width.  A pipeline stage holds the halo run of one slab of SLAB channels:
// 32 (128-byte rows, SWIZZLE_128B) or 16 (64-byte rows, SWIZZLE_64B), the latter
// for layers whose filter bank leaves no room for two 32-channel stages.  The
// weights keep their 32-row blocks either way; a 16-channel slab reads the upper
// or lower 16 rows of its block.
//
// What bounds this kernel.  A 128 x N x 8 TF32 MMA reads 4 KB of A and N/32 KB of
// B from shared memory, which delivers 128 B per clock: N = 64 takes 48 clocks
// (measured; 32 would be the arithmetic), N = 128 takes 64, only N = 256 is bound
// by the tensor pipe itself (128).  With F = 64 this kernel therefore runs at 2/3
// of the tensor peak at best, and the halo copies share the same shared-memory
// bandwidth.  Measured on 32x56x56x64 -> 64, 3x3 (841 tiles over 148 SMs): 6.9 us
// without any MMA (launch, filter bank, copies, stores), 18.3 us with the MMAs
// alone, 22.6 us in full.
//
// Two issuing threads.  One thread cannot issue tcgen05.mma faster than about one
// per 55 clocks (measured, whatever N), and the descriptor arithmetic of this loop
// raises that to ~75.  With DUAL, warps 1 and 2 each issue half of the taps of
// every slab into an accumulator of their own, and the epilogue adds the two: the
// shared-memory feed, not the issue loop, sets the pace, and the result does not
// depend on how the two instruction streams interleave.
#pragma once
#include "gemm_tf32.cuh"

namespace xtc {

// Optional per-CTA event trace (clock64 stamps) for kernel studies: compiled in only with
// -DXTC_TRACE, where the host sets g_halo_trace to a device buffer of
// [CTA][role 0..3][XTC_TRACE_EVENTS] stamps.
#ifdef XTC_TRACE
#define XTC_TRACE_EVENTS 128
static __device__ long long* g_halo_trace = nullptr;  // one translation unit includes this header
#define XTC_TRACE_DECL(role) int _tn = 0; long long* _tb = g_halo_trace ? g_halo_trace + ((static_cast<size_t>(blockIdx.x) * 4 + (role)) * XTC_TRACE_EVENTS) : nullptr
#define XTC_TRACE_MARK() do { if (_tb && _tn < XTC_TRACE_EVENTS) _tb[_tn++] = clock64(); } while (0)
#else
#define XTC_TRACE_DECL(role)
#define XTC_TRACE_MARK()
#endif

struct ConvHaloParams {
  float* Y;
  int* status;
  long long Q;            // B * Hp * Wp positions
  int tiles;              // ceil(Q / 128), or / 256 in the CTA-pair kernel
  int Hp, Wp, OH, OW, F;
  int nslab;              // ceil(C / SLAB): halo copies (pipeline stages) per tile
  int nblk;               // ceil(C / 32): 32-channel weight blocks per tap
  int C;
  int taps, S;            // R*S, S
  int pad_left, pad_top;
  int stage_bytes;        // P * SLAB * 4 rounded up to 1024: distance between stages
  int stage_tx;           // P * SLAB * 4: bytes one halo copy delivers
  int stages;
  int relu;
  float relu_threshold;
  // streamed-weights kernel (conv2d_halo_stream.cuh) only
  int ntiles_n;           // filter tiles of 128
  int wts_offset;         // where a stage's weights start (the halo slab rounded up to 1024 bytes)
  int wts_tx;             // bytes of weights one CTA fetches per stage: taps * 64 * 128
  // the same kernel with the (work item, channel slab) units dealt out evenly to the CTA pairs
  float* sk_partials;     // NULL = whole work items, round-robin; else [pair][CTA][warp][32 rows x 128 columns]
  int* sk_flags;          // [pair][CTA][warp]: 1 = that warp's partial is in place (its reader clears it)
};

constexpr int HALO_THREADS = 224;  // producer, two MMA issuers, four epilogue warps

template <int BN, bool DUAL, int SLAB>
__global__ void __launch_bounds__(HALO_THREADS, 1)
conv2d_halo_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const ConvHaloParams p) {
  using namespace dev;
  constexpr int NACC = DUAL ? 2 : 1;  // accumulators per tile, one per issuing thread
  constexpr uint32_t TMEM_COLS = 2 * NACC * BN < 32 ? 32 : 2 * NACC * BN;
  static_assert(TMEM_COLS <= 512, "accumulators do not fit in TMEM");
  static_assert(SLAB == 16 || SLAB == 32, "slabs are 16 or 32 channels wide");
  constexpr int ROW = SLAB * 4;     // bytes per pixel row of a stage
  constexpr int WBLOCK = BN * 128;  // bytes of weights per (tap, block): 32 k-rows x BN columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* wts = smem;  // taps * nslab * WBLOCK
  uint8_t* ring = wts + static_cast<size_t>(p.taps) * p.nblk * WBLOCK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(p.stages) * p.stage_bytes);
  uint64_t* full = bars;           // [stages]
  uint64_t* empty = bars + 8;      // [stages]
  uint64_t* acc_full = bars + 16;  // [2]
  uint64_t* acc_empty = bars + 18; // [2]
  uint64_t* wbar = bars + 20;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NACC);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], NACC);
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
    // The first tile's halo copies go out before anything else: they come from DRAM (the
    // input of a step is cold) while the filter bank comes from L2, and the first MMA needs
    // both.  Every stage is free at this point, so nothing is waited for.
    const int first_slabs = p.nslab < p.stages ? p.nslab : p.stages;
    auto issue_halo = [&](int tile, int slab, int stage) {
      const long long q0 = static_cast<long long>(tile) * BM;
      const int img = static_cast<int>(q0 / plane);
      const int rem = static_cast<int>(q0 - static_cast<long long>(img) * plane);
      const int ih = rem / p.Wp - p.pad_top;
      const int iw = rem % p.Wp - p.pad_left;
      mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(p.stage_tx));
      tma_load_im2col_4d(ring + static_cast<size_t>(stage) * p.stage_bytes, &tmX, &full[stage],
                         slab * SLAB, iw, ih, img, 0, 0);
    };
    if (lane == 0) {
      for (int slab = 0; slab < first_slabs; ++slab) issue_halo(blockIdx.x, slab, slab);
      // The filter bank, once: one thread announces the bytes, then every lane issues its
      // share of the copies (issuing them all from one thread takes longer than they take to
      // arrive).
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
      XTC_TRACE_DECL(0);
      XTC_TRACE_MARK();  // start
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;  // copies counted so far; the first `first_slabs` are already out
      for (int tile = blockIdx.x; tile < p.tiles && !failed; tile += gridDim.x) {
        for (int slab = 0; slab < p.nslab; ++slab, ++issued) {
          if (issued >= first_slabs) {
            if (!mbar_wait(&empty[stage], phase ^ 1)) {
              atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_EMPTY);
              failed = true;
              break;
            }
            XTC_TRACE_MARK();  // stage free: load issued
            issue_halo(tile, slab, stage);
          }
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp <= 2) {
    // ------------------------------ MMA issuers ------------------------------
    const int w = warp - 1;
    if (lane == 0 && w < NACC) {
      constexpr uint32_t idesc = umma_idesc_tf32(BM, BN, false, true);
      // this thread's share of the taps
      const int t0 = DUAL ? (w == 0 ? 0 : (p.taps + 1) / 2) : 0;
      const int t1 = DUAL ? (w == 0 ? (p.taps + 1) / 2 : p.taps) : p.taps;
      const int r0 = t0 / p.S, s0 = t0 - r0 * p.S;
      XTC_TRACE_DECL(1 + w);
      XTC_TRACE_MARK();  // start
      if (!mbar_wait(wbar, 0)) {
        atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
        failed = true;
      }
      XTC_TRACE_MARK();  // bank landed
      const uint32_t w0 = smem_u32(wts) + static_cast<uint32_t>(t0) * p.nblk * WBLOCK;
      // A: K-major rows of ROW bytes, 8-row swizzle atoms
      const uint32_t a_hi = umma_desc_hi(8 * ROW, static_cast<uint32_t>(SLAB == 32 ? UMMA_SWIZZLE_128B
                                                                                  : UMMA_SWIZZLE_64B));
      const uint32_t b_hi = umma_desc_hi(512, static_cast<uint32_t>(UMMA_SWIZZLE_128B_BASE32B));
      const uint32_t b_step = static_cast<uint32_t>(p.nblk) * (WBLOCK >> 4);
      constexpr uint32_t PIX = ROW >> 4;                               // one pixel row, >> 4
      const uint32_t row_step = static_cast<uint32_t>(p.Wp) * PIX;  // one image row down
      const uint32_t a_first = static_cast<uint32_t>(r0) * row_step;
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
        const uint32_t d_tmem = tmem_base + (acc * NACC + w) * BN;
        for (int slab = 0; slab < p.nslab; ++slab) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
            failed = true;
            break;
          }
          XTC_TRACE_MARK();  // slab landed
          const uint32_t sA = smem_u32(ring + static_cast<size_t>(stage) * p.stage_bytes);
          uint32_t a_row = umma_desc_lo(sA, 16) + a_first;  // tap (r, 0)
          // k rows [slab * SLAB, +SLAB) of the filter bank: block slab*SLAB/32, 128 B per k row
          const uint32_t k0 = static_cast<uint32_t>(slab) * SLAB;
          uint32_t b_lo = umma_desc_lo(w0 + (k0 >> 5) * WBLOCK + (k0 & 31u) * 128u, 4096);
          uint32_t first = slab == 0 ? 0u : 1u;
          for (int tap = t0, s = s0; tap < t1; ++tap) {
            const uint32_t a_lo = a_row + static_cast<uint32_t>(s) * PIX;
#pragma unroll
            for (int kk = 0; kk < SLAB / 8; ++kk) {
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
      const long long q = static_cast<long long>(tile) * BM + quad * 32 + lane;
      const int img = static_cast<int>(q / plane);
      const int rem = static_cast<int>(q - static_cast<long long>(img) * plane);
      const int oh = rem / p.Wp;
      const int ow = rem - oh * p.Wp;
      const bool valid = q < p.Q && oh < p.OH && ow < p.OW;
      float* dst = p.Y + ((static_cast<long long>(img) * p.OH + oh) * p.OW + ow) * p.F;
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
