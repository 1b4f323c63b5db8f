// Shared device/host helpers for the sm_100a kernels of libxtc_cuda:
// error reporting, bounded mbarrier waits, TMA and tcgen05 PTX wrappers, and
// the UMMA shared-memory / instruction descriptor encodings.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/xtc_cuda.h"

namespace xtc {

// ---------------------------------------------------------------------------
// Host side: thread-local last-error string and status helpers
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
const char* get_error();

#define XTC_CUDA_CHECK(expr)                                                        \
  do {                                                                              \
    cudaError_t _e = (expr);                                                        \
    if (_e != cudaSuccess) {                                                        \
      ::xtc::set_error("%s:%d: %s failed: %s", __FILE__, __LINE__, #expr,           \
                       cudaGetErrorString(_e));                                     \
      return XTC_CUDA_ERR_RUNTIME;                                                  \
    }                                                                               \
  } while (0)

#define XTC_REQUIRE(cond, ...)                                                      \
  do {                                                                              \
    if (!(cond)) {                                                                  \
      ::xtc::set_error(__VA_ARGS__);                                                \
      return XTC_CUDA_ERR_INVALID;                                                  \
    }                                                                               \
  } while (0)

// Per-device word the kernels write when a bounded wait gives up.  Kernels never
// trap; the host reads this word after synchronising (xtc_cuda_device_status).
int* device_status_word(int dev);
// The status word of the allocation-free GEMM (it lives in the library image, see
// gemm_tf32.cu): reads it into *status and clears it when set.  0 when that entry point
// has not been used on `dev` yet.  Allocates nothing.
int noalloc_status_fetch_and_clear(int dev, int* status);

// Tensor-map encoders resolved through cudaGetDriverEntryPoint, so that the
// library has no link-time dependency on libcuda and loads on a machine
// without a driver.
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*encode_im2col_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                     cuuint32_t, cuuint32_t, const cuuint32_t*,
                                     CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn get_encode_tiled();
encode_im2col_fn get_encode_im2col();

// Rank-4 fp32 map without swizzle: dims / box innermost first, strides (in floats) of dims 1..3.
// Returns false (no error recorded) when the driver rejects the geometry.
bool make_tmap_4d_plain(CUtensorMap* map, const void* base, const uint64_t dims[4],
                        const uint64_t strides[3], const uint32_t box[4]);
// 2-D fp32 tiled map over a row-major [rows, cols] matrix with leading
// dimension ld (elements).  box = {box_cols, box_rows}.
int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle swizzle);

int sm_count(int dev);

// Kernel, tile and split-K factor the library picks for a TF32 contraction M x N x K
// whose caller named none of them (cost model in gemm_tf32.cu).
struct AutoChoice {
  int tile_m, tile_n, tile_k, split_k;
};
// `cluster_cap[s]` (s = 2 .. 8) = clusters of s single-CTA GEMM blocks the
// device runs at once (cluster_capacity), NULL = do not consider a split inside a cluster.
// `pair_tail_ok` = the CTA-pair kernel may cut the tiles of a partly idle round along K (the
// GEMM's pair kernel does, given a workspace; the convolution's does not).
AutoChoice choose_tf32_default(int64_t M, int64_t N, int64_t K, int sms, bool pair_ok,
                               bool split_ok, const int* cluster_cap = nullptr,
                               bool pair_tail_ok = true);
int cluster_capacity(int dev, int size);
// Pieces (8 down to 2, or 1 = do not split) a cluster split of `k_blocks` K stages runs with
// when `want` were asked for: the largest count not above `want` whose pieces, of
// ceil(k_blocks / pieces) stages each, are all non-empty.
inline int cluster_pieces(int k_blocks, int want) {
  for (int s = 8; s >= 2; --s) {
    if (s > want) continue;
    const int per = (k_blocks + s - 1) / s;
    if ((s - 1) * per < k_blocks) return s;
  }
  return 1;
}

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------
namespace dev {

enum : int {
  STATUS_OK = 0,
  STATUS_WAIT_TIMEOUT_LOAD = 1,   // consumer never saw a TMA stage arrive
  STATUS_WAIT_TIMEOUT_EMPTY = 2,  // producer never saw a stage released
  STATUS_WAIT_TIMEOUT_ACC = 3,    // epilogue never saw the accumulator commit
  STATUS_WAIT_TIMEOUT_DRAIN = 4,  // MMA issuer never saw the accumulator drained
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: spins on the barrier phase for at most `limit_ns` of wall time, then
// gives up and returns false.  The caller records a status code and unwinds.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0x3ff) == 0x3ff) {
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
}
// The limit every kernel of the library uses: about 2 s.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  return mbar_wait_limit(bar, parity, 2000000000ull);
}

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with launch_overlapped() may start while the previous kernel
// of its stream is still finishing; its CTAs run their prologue (barriers, TMEM,
// descriptor prefetch) and then wait here until that kernel's memory is complete.
// Without the launch attribute both calls do nothing.
__device__ __forceinline__ void grid_dependency_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- TMA -----------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(void* dst, const CUtensorMap* m, uint64_t* bar,
                                                   int c, int w, int h, int n, uint16_t off_w,
                                                   uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n),
      "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
// L2 eviction policy for data that is written once and not read again by this kernel.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* m, const void* src, int x,
                                                  int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::
          "l"(reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(src)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// The same copies with an L2 eviction hint (data that passes through once).
__device__ __forceinline__ void tma_load_4d_hint(void* dst, const CUtensorMap* m, uint64_t* bar,
                                                 int c0, int c1, int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d_hint(const CUtensorMap* m, const void* src, int c0,
                                                  int c1, int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4, %5}], [%1], %6;" ::
          "l"(reinterpret_cast<uint64_t>(m)),
      "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05 / TMEM --------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], TF32 inputs, FP32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row
// (lane_base + i), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- CTA pairs (cta_group::2): two SMs share one MMA ------------------------
// Address, in the cluster's shared window, of the same shared-memory offset in
// the CTA with rank `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float4 ld_shared_cluster_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
// Sums, in piece order, the float4 at the same shared-memory offset of the first PIECES CTAs of
// the cluster, for two offsets at once: all 2 * PIECES reads are issued before the first add.
template <int PIECES>
__device__ __forceinline__ void sum_cluster_pieces(uint32_t addr_a, uint32_t addr_b, float4& sum_a,
                                                   float4& sum_b) {
  float4 va[PIECES], vb[PIECES];
#pragma unroll
  for (int piece = 0; piece < PIECES; ++piece) {
    va[piece] = ld_shared_cluster_f4(map_to_cta(addr_a, piece));
    vb[piece] = ld_shared_cluster_f4(map_to_cta(addr_b, piece));
  }
  sum_a = make_float4(0.f, 0.f, 0.f, 0.f);
  sum_b = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int piece = 0; piece < PIECES; ++piece) {
    sum_a.x += va[piece].x; sum_a.y += va[piece].y; sum_a.z += va[piece].z; sum_a.w += va[piece].w;
    sum_b.x += vb[piece].x; sum_b.y += vb[piece].y; sum_b.z += vb[piece].z; sum_b.w += vb[piece].w;
  }
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
// TMA load into this CTA's shared memory that reports its bytes to the mbarrier at
// `bar_addr`, which may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, uint32_t bar_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* m, uint32_t bar_addr,
                                                 int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d_pair(void* dst, const CUtensorMap* m,
                                                        uint32_t bar_addr, int c, int w, int h,
                                                        int n, uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_addr), "r"(c), "r"(w), "r"(h), "r"(n),
      "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// Arrive on the mbarrier at `bar_addr` (any CTA of the pair) once all MMAs issued
// so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_addr)
               : "memory");
}
// 256 x N x 8 MMA over the pair: A rows and B columns are split between the CTAs.
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- 256-bit global store ----------------------------------------------------
// Eight consecutive floats in one instruction: a whole 32-byte sector per lane, so a thread
// that owns a row of a tile never leaves a half-written sector for L2 to merge.  The address
// must be 32-byte aligned.
__device__ __forceinline__ void st_global_f8(float* addr, const uint32_t* r) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(addr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// ---- NVLink multicast --------------------------------------------------------
// One 128-bit store to a multicast address: the switch writes it to the same offset of every
// GPU memory bound to the multicast object (this GPU's included).
__device__ __forceinline__ void multimem_st_f4(float* mc_addr, float4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// ---- UMMA descriptors ------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address, leading/stride byte
// offsets (all >> 4), descriptor version 1 (sm_100), swizzle mode in bits 61..63.
enum : uint64_t {
  UMMA_SWIZZLE_NONE = 0,
  UMMA_SWIZZLE_128B_BASE32B = 1,  // 128-byte span, 32-byte atoms: MN-major 32-bit operands
  UMMA_SWIZZLE_128B = 2,
  UMMA_SWIZZLE_64B = 4,
};
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint64_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;
  d |= swizzle << 61;
  return d;
}
// The same descriptor as two 32-bit halves.  The issuing thread builds the halves
// once per pipeline stage and then only adds (byte offset >> 4) to the low half
// for every MMA: the start address sits in its low 14 bits, and one thread has
// to issue an MMA every few dozen cycles, so the per-MMA instruction count matters.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3ffff) >> 4) | (((lbo_bytes >> 4) & 0x3fff) << 16);
}
__device__ __forceinline__ uint32_t umma_desc_hi(uint32_t sbo_bytes, uint32_t swizzle) {
  return ((sbo_bytes >> 4) & 0x3fff) | (1u << 14) | (swizzle << 29);
}
__device__ __forceinline__ uint64_t umma_desc_pack(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor for kind::tf32, fp32 accumulate.  a_mn / b_mn select an
// MN-major (transposed) operand; M and N are the instruction tile extents.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, bool a_mn, bool b_mn) {
  return (1u << 4)                            // D format: F32
         | (2u << 7)                          // A format: TF32
         | (2u << 10)                         // B format: TF32
         | (static_cast<uint32_t>(a_mn) << 15)
         | (static_cast<uint32_t>(b_mn) << 16)
         | (static_cast<uint32_t>(N >> 3) << 17)
         | (static_cast<uint32_t>(M >> 4) << 24);
}

}  // namespace dev

// Bounded wait (about 2 s) for a flag in global memory that another CTA sets.
__device__ __forceinline__ bool wait_flag_set(int* flag) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (atomicAdd(flag, 0) != 0) return true;
    if ((it & 0xff) == 0xff) {
      const uint64_t now = dev::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) return false;
    }
  }
}

// Launch with programmatic stream serialisation: the kernel may begin before its
// predecessor in the stream has drained (see dev::grid_dependency_sync).
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped_clustered(void (*kernel)(KArgs...), unsigned grid, unsigned cluster,
                                        unsigned block, size_t smem, cudaStream_t stream,
                                        Args&&... args) {
  cudaLaunchConfig_t lc;
  memset(&lc, 0, sizeof(lc));
  lc.gridDim = dim3(grid, 1, 1);
  lc.blockDim = dim3(block, 1, 1);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  memset(attr, 0, sizeof(attr));
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;  // `cluster` consecutive CTAs form a cluster
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = cluster > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&lc, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  return launch_overlapped_clustered(kernel, grid, 1u, block, smem, stream,
                                     static_cast<Args&&>(args)...);
}
#endif  // __CUDACC__

}  // namespace xtc
