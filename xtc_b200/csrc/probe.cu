// Tensor-pipe peak probe: every SM issues a long chain of 128x256x8 TF32 MMAs on
// operands that stay in shared memory (no global traffic), so the measured rate
// is the issue/compute limit of tcgen05.mma kind::tf32.  Returns FMA/s, the unit
// of the reference's CPU probe (evaluate_flops).
#include "common.cuh"

namespace xtc {
using namespace dev;

template <int M, int N>
__global__ void __launch_bounds__(128, 1) tf32_peak_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int A_BYTES = 128 * 128, B_BYTES = 256 * 128;  // room for the largest shape
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + A_BYTES + B_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x)
    reinterpret_cast<float*>(smem)[i] = 0.f;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  fence_proxy_async();
  if (threadIdx.x < 32) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_tf32(M, N, false, false);
    const uint32_t sA = smem_u32(smem), sB = sA + A_BYTES;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        umma_tf32(tmem, umma_smem_desc(sA + kk * 32, 16, 1024, UMMA_SWIZZLE_128B),
                  umma_smem_desc(sB + kk * 32, 16, 1024, UMMA_SWIZZLE_128B), idesc, (it | kk) != 0);
      }
    }
    tc_commit(bar);
    if (!mbar_wait(bar, 0)) atomicCAS(status, 0, STATUS_WAIT_TIMEOUT_ACC);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}
}  // namespace xtc

using namespace xtc;

namespace {
template <int M, int N>
int measure_rate(double* fma_per_second) {
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  int* status = device_status_word(dev);
  XTC_REQUIRE(status != nullptr, "peak_fma: device status word unavailable");
  const int smem = 1024 + 128 * 128 + 256 * 128 + 64;
  XTC_CUDA_CHECK(cudaFuncSetAttribute(tf32_peak_kernel<M, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int sms = sm_count(dev);
  const int iters = 4096;
  cudaEvent_t e0, e1;
  XTC_CUDA_CHECK(cudaEventCreate(&e0));
  XTC_CUDA_CHECK(cudaEventCreate(&e1));
  double best = 0.0;
  for (int rep = 0; rep < 5; ++rep) {
    cudaEventRecord(e0, nullptr);
    tf32_peak_kernel<M, N><<<sms, 128, smem, nullptr>>>(iters, status);
    cudaEventRecord(e1, nullptr);
    XTC_CUDA_CHECK(cudaGetLastError());
    XTC_CUDA_CHECK(cudaEventSynchronize(e1));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    const double fma = static_cast<double>(sms) * iters * 4.0 * M * N * 8.0;
    if (ms > 0.f && rep > 0) best = fma / (ms * 1e-3) > best ? fma / (ms * 1e-3) : best;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *fma_per_second = best;
  return XTC_CUDA_OK;
}
}  // namespace

extern "C" int xtc_cuda_peak_fma(const char* dtype, double* fma_per_second) {
  XTC_REQUIRE(dtype && fma_per_second, "peak_fma: NULL argument");
  XTC_REQUIRE(strcmp(dtype, "float32") == 0, "peak_fma: only float32 (TF32 tensor pipe) is probed, got %s", dtype);
  return measure_rate<128, 256>(fma_per_second);
}

extern "C" int xtc_cuda_mma_rate(int tile_m, int tile_n, double* fma_per_second) {
  XTC_REQUIRE(fma_per_second != nullptr, "mma_rate: NULL argument");
#define XTC_RATE_CASE(M_, N_) \
  if (tile_m == M_ && tile_n == N_) return measure_rate<M_, N_>(fma_per_second);
  XTC_RATE_CASE(64, 64) XTC_RATE_CASE(64, 128) XTC_RATE_CASE(64, 256)
  XTC_RATE_CASE(128, 64) XTC_RATE_CASE(128, 128) XTC_RATE_CASE(128, 256)
#undef XTC_RATE_CASE
  set_error("mma_rate: tile %d x %d is not an MMA shape of one CTA (rows 64 or 128, columns 64, 128 or 256)",
            tile_m, tile_n);
  return XTC_CUDA_ERR_INVALID;
}
