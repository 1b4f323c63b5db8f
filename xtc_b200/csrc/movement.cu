// Bandwidth-bound kernels: transpose, constant pad / crop, relu and the
// hi/lo operand split of the 3xTF32 mode.  All are single pass (each input
// element read once, each output element written once) with 128-bit accesses
// wherever alignment allows, and bit-exact data movement.
#include "common.cuh"

namespace xtc {

// ---------------------------------------------------------------------------
// relu / split: grid-stride, float4
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
relu_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n, float thr) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t n4 = n >> 2;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float4* y4 = reinterpret_cast<float4*>(y);
  int64_t i = tid;
  // four independent 128-bit loads in flight per thread before the first store
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = __ldcs(x4 + i + u * stride);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      v[u].x = fmaxf(v[u].x, thr); v[u].y = fmaxf(v[u].y, thr);
      v[u].z = fmaxf(v[u].z, thr); v[u].w = fmaxf(v[u].w, thr);
      __stcs(y4 + i + u * stride, v[u]);
    }
  }
  for (; i < n4; i += stride) {
    float4 v = __ldcs(x4 + i);
    v.x = fmaxf(v.x, thr); v.y = fmaxf(v.y, thr); v.z = fmaxf(v.z, thr); v.w = fmaxf(v.w, thr);
    __stcs(y4 + i, v);
  }
  for (int64_t j = (n4 << 2) + tid; j < n; j += stride) y[j] = fmaxf(x[j], thr);
}

__global__ void __launch_bounds__(256)
relu_f32_scalar_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n, float thr) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = fmaxf(x[i], thr);
}

__device__ __forceinline__ float round_tf32(float v) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo,
                  int64_t n) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t n4 = n >> 2;
  for (int64_t i = tid; i < n4; i += stride) {
    float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
    float4 h, l;
    h.x = round_tf32(v.x); h.y = round_tf32(v.y); h.z = round_tf32(v.z); h.w = round_tf32(v.w);
    l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
    reinterpret_cast<float4*>(hi)[i] = h;
    reinterpret_cast<float4*>(lo)[i] = l;
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
    float h = round_tf32(x[i]);
    hi[i] = h;
    lo[i] = x[i] - h;
  }
}

// ---------------------------------------------------------------------------
// transpose
// ---------------------------------------------------------------------------
struct TransposeDims {
  int ndim;               // rank after merging axes
  int64_t in_shape[XTC_CUDA_MAX_DIMS];
  int64_t in_stride[XTC_CUDA_MAX_DIMS];   // input strides (elements), indexed by input axis
  int64_t out_shape[XTC_CUDA_MAX_DIMS];   // out_shape[d] = in_shape[axes[d]]
  int64_t out_in_stride[XTC_CUDA_MAX_DIMS];  // input stride of the axis that output dim d walks
  int axes[XTC_CUDA_MAX_DIMS];
};

// Batched 2-D tile transpose.  The input's innermost axis (length C, stride 1)
// lands at output dim `oc`; the output's innermost dim walks input axis `ar`
// (length R, input stride rs).  A 64x64 tile is read with 128-bit loads along C,
// transposed through padded shared memory, and written with 128-bit stores
// along R.  Remaining dims form the batch.
struct Tile2DParams {
  int64_t R, C;             // tile-plane extents (R: output-contiguous, C: input-contiguous)
  int64_t in_r_stride;      // input stride of R axis
  int64_t out_c_stride;     // output stride of C axis
  int nbatch_dims;
  int64_t batch_shape[XTC_CUDA_MAX_DIMS];
  int64_t batch_in_stride[XTC_CUDA_MAX_DIMS];
  int64_t batch_out_stride[XTC_CUDA_MAX_DIMS];
  int64_t tiles_r, tiles_c;
  int vec_in, vec_out;      // 128-bit access legal on the input / output side
};

template <int TILE>
__global__ void __launch_bounds__(256)
transpose_tile_kernel(const float* __restrict__ x, float* __restrict__ y, Tile2DParams p) {
  __shared__ float tile[TILE][TILE + 1];
  int64_t b = blockIdx.x;
  const int64_t tc = b % p.tiles_c; b /= p.tiles_c;
  const int64_t tr = b % p.tiles_r; b /= p.tiles_r;
  int64_t in_off = 0, out_off = 0;
  for (int d = p.nbatch_dims - 1; d >= 0; --d) {
    const int64_t i = b % p.batch_shape[d];
    b /= p.batch_shape[d];
    in_off += i * p.batch_in_stride[d];
    out_off += i * p.batch_out_stride[d];
  }
  const int64_t r0 = tr * TILE, c0 = tc * TILE;
  const float* src = x + in_off + r0 * p.in_r_stride + c0;
  float* dst = y + out_off + c0 * p.out_c_stride + r0;
  const int64_t nr = (p.R - r0) < TILE ? (p.R - r0) : TILE, nc = (p.C - c0) < TILE ? (p.C - c0) : TILE;
  constexpr int V = TILE / 4;  // float4 per tile row

  if (p.vec_in && nc == TILE) {
    for (int i = threadIdx.x; i < TILE * V; i += 256) {
      const int r = i / V, c4 = i % V;
      if (r < nr) {
        float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * p.in_r_stride) + c4);
        tile[r][c4 * 4 + 0] = v.x; tile[r][c4 * 4 + 1] = v.y;
        tile[r][c4 * 4 + 2] = v.z; tile[r][c4 * 4 + 3] = v.w;
      }
    }
  } else {
    for (int i = threadIdx.x; i < TILE * TILE; i += 256) {
      const int r = i / TILE, c = i % TILE;
      if (r < nr && c < nc) tile[r][c] = src[r * p.in_r_stride + c];
    }
  }
  __syncthreads();
  if (p.vec_out && nr == TILE) {
    for (int i = threadIdx.x; i < TILE * V; i += 256) {
      const int c = i / V, r4 = i % V;
      if (c < nc) {
        float4 v = make_float4(tile[r4 * 4 + 0][c], tile[r4 * 4 + 1][c], tile[r4 * 4 + 2][c],
                               tile[r4 * 4 + 3][c]);
        __stcs(reinterpret_cast<float4*>(dst + c * p.out_c_stride) + r4, v);
      }
    }
  } else {
    for (int i = threadIdx.x; i < TILE * TILE; i += 256) {
      const int c = i / TILE, r = i % TILE;
      if (r < nr && c < nc) dst[c * p.out_c_stride + r] = tile[r][c];
    }
  }
}

// The same tile transpose with the global traffic handed to TMA: a persistent CTA
// keeps three 64x64 input tiles in flight (bulk tensor loads, zero-filled at the
// edges) and two output tiles draining (bulk tensor stores, clipped at the edges),
// and its threads only move data between the two shared-memory tiles.  Both tiles
// are dense, so lane l of a warp walks a diagonal of its 32x32 block: element
// (l, (l+i) mod 32) in step i, whose bank is (l+i) mod 32 on the read side and l on
// the write side; no padding, no conflicts.
constexpr int TT = 64;
constexpr int TT_STAGES = 3;
constexpr int TT_TILE_BYTES = TT * TT * 4;
constexpr int TT_SMEM = 1024 + (TT_STAGES + 2) * TT_TILE_BYTES + 64;

struct TmaTransposeParams {
  long long tiles_c, tiles_r, b0;  // tile grid: along the input's inner axis, its row axis, first batch axis
  long long total;                 // tiles_c * tiles_r * b0 * b1
  int* status;
};

__global__ void __launch_bounds__(256, 2)
transpose_tma_kernel(const __grid_constant__ CUtensorMap tmIn,
                     const __grid_constant__ CUtensorMap tmOut, const TmaTransposeParams p) {
  using namespace dev;
  extern __shared__ uint8_t tt_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tt_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* in_tiles = reinterpret_cast<float*>(smem);
  float* out_tiles = reinterpret_cast<float*>(smem + TT_STAGES * TT_TILE_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (TT_STAGES + 2) * TT_TILE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // every element is read once and written once: both sides are marked evict-first in L2
  const uint64_t once = l2_policy_evict_first();
  auto coords = [&](long long t, int& c0, int& r0, int& i0, int& i1) {
    const long long tc = t % p.tiles_c; t /= p.tiles_c;
    const long long tr = t % p.tiles_r; t /= p.tiles_r;
    c0 = static_cast<int>(tc) * TT;
    r0 = static_cast<int>(tr) * TT;
    i0 = static_cast<int>(t % p.b0);
    i1 = static_cast<int>(t / p.b0);
  };
  auto load = [&](long long t, int stage) {
    int c0, r0, i0, i1;
    coords(t, c0, r0, i0, i1);
    mbar_arrive_expect_tx(&full[stage], TT_TILE_BYTES);
    tma_load_4d_hint(in_tiles + stage * (TT * TT), &tmIn, &full[stage], c0, r0, i0, i1, once);
  };

  if (tid == 0) {
    prefetch_tmap(&tmIn);
    prefetch_tmap(&tmOut);
    for (int s = 0; s < TT_STAGES; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
  }
  __syncthreads();
  grid_dependency_sync();
  const long long first = blockIdx.x, step = gridDim.x;
  if (tid == 0)
    for (int s = 0; s < TT_STAGES; ++s)
      if (first + s * step < p.total) load(first + s * step, s);

  const int blk = warp & 3;                 // which 32x32 block of the tile
  const int br = (blk >> 1) * 32, bc = (blk & 1) * 32;
  const int i_lo = (warp >> 2) * 16;        // which half of the 32 diagonal steps
  int stage = 0, o = 0;
  uint32_t phase = 0;
  bool gave_up = false;
  for (long long t = first; t < p.total; t += step) {
    int failed = mbar_wait(&full[stage], phase) ? 0 : 1;
    if (tid == 0) tma_store_wait_read<1>();  // the store issued two tiles ago has read out_tiles[o]
    if (__syncthreads_or(failed)) {
      if (tid == 0) atomicCAS(p.status, 0, STATUS_WAIT_TIMEOUT_LOAD);
      gave_up = true;
      break;
    }
    const float* src = in_tiles + stage * (TT * TT);
    float* dst = out_tiles + o * (TT * TT);
    const int r = br + lane;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int c = bc + ((lane + i_lo + i) & 31);
      dst[c * TT + r] = src[r * TT + c];
    }
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
      int c0, r0, i0, i1;
      coords(t, c0, r0, i0, i1);
      tma_store_4d_hint(&tmOut, dst, r0, c0, i0, i1, once);
      tma_store_commit();
      const long long next = t + TT_STAGES * step;
      if (next < p.total) load(next, stage);
    }
    if (++stage == TT_STAGES) {
      stage = 0;
      phase ^= 1;
    }
    o ^= 1;
  }
  if (gave_up) {  // let copies still in flight land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  if (tid == 0) tma_store_wait_all<0>();
}

// Permutation that keeps the innermost axis: rows of `inner` contiguous floats
// are copied whole; `vec` floats (4 or 1) per thread.
struct RowCopyParams {
  int ndim;  // outer dims (output order)
  int64_t out_shape[XTC_CUDA_MAX_DIMS];
  int64_t in_stride[XTC_CUDA_MAX_DIMS];
  int64_t inner;   // innermost extent in units of `vec` floats
  int64_t total;   // total units
};

template <typename T>
__global__ void __launch_bounds__(256)
permute_rows_kernel(const T* __restrict__ x, T* __restrict__ y, RowCopyParams p, int64_t in_unit) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total;
       i += stride) {
    int64_t rem = i / p.inner;
    const int64_t col = i - rem * p.inner;
    int64_t off = 0;
    for (int d = p.ndim - 1; d >= 0; --d) {
      const int64_t q = rem / p.out_shape[d];
      off += (rem - q * p.out_shape[d]) * p.in_stride[d];
      rem = q;
    }
    y[i] = x[off / in_unit + col];
  }
}

// ---------------------------------------------------------------------------
// pad / crop: output indexed, one pass
// ---------------------------------------------------------------------------
struct PadParams {
  int ndim;
  int64_t out_shape[XTC_CUDA_MAX_DIMS];   // innermost in units of VEC floats
  int64_t in_shape[XTC_CUDA_MAX_DIMS];
  int64_t in_stride[XTC_CUDA_MAX_DIMS];   // in units of VEC floats
  int64_t lo[XTC_CUDA_MAX_DIMS];
  int64_t total;
  float value;
};

template <typename T>
__device__ __forceinline__ T splat(float v);
template <> __device__ __forceinline__ float splat<float>(float v) { return v; }
template <> __device__ __forceinline__ float4 splat<float4>(float v) { return make_float4(v, v, v, v); }

// One output row (the innermost axis, after axes without padding have been merged into
// their outer neighbours) per `lanes` threads: the row's position along the outer axes is
// decoded once per row, the copy along the row needs no division.  lanes is a power of two
// <= 256; a block handles 256 / lanes rows at a time.
template <typename T>
__global__ void __launch_bounds__(256)
pad_kernel(const T* __restrict__ x, T* __restrict__ y, PadParams p, int lane_shift, int64_t rows,
           int64_t chunks, int64_t chunk_width) {
  const int lanes = 1 << lane_shift;
  const int rows_per_block = 256 >> lane_shift;
  const int lane = threadIdx.x & (lanes - 1);
  const int sub = threadIdx.x >> lane_shift;
  const T fill = splat<T>(p.value);
  const int last = p.ndim - 1;
  const int64_t width = p.out_shape[last], in_width = p.in_shape[last], lo = p.lo[last];
  // work item = (row, chunk of chunk_width columns): long rows are shared by several groups
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * rows_per_block + sub; item < rows * chunks;
       item += static_cast<int64_t>(gridDim.x) * rows_per_block) {
    const int64_t row = item / chunks;
    const int64_t col_lo = (item - row * chunks) * chunk_width;
    const int64_t col_hi = col_lo + chunk_width < width ? col_lo + chunk_width : width;
    int64_t rem = row, off = 0;
    bool inside = true;
    for (int d = last - 1; d >= 0; --d) {
      const int64_t q = rem / p.out_shape[d];
      const int64_t c = (rem - q * p.out_shape[d]) - p.lo[d];
      rem = q;
      inside = inside && c >= 0 && c < p.in_shape[d];
      off += c * p.in_stride[d];
    }
    T* dst = y + row * width;
    const T* src = x + off - lo;  // src[col] is the input element under output column col
    if (!inside) {
      for (int64_t col = col_lo + lane; col < col_hi; col += lanes) __stcs(dst + col, fill);
      continue;
    }
    const int64_t hi_edge = lo + in_width;
    int64_t col = col_lo + lane;
    for (; col + 3 * lanes < col_hi; col += 4 * lanes) {
      T v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t c = col + u * lanes;
        v[u] = (c >= lo && c < hi_edge) ? __ldcs(src + c) : fill;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) __stcs(dst + col + u * lanes, v[u]);
    }
    for (; col < col_hi; col += lanes)
      __stcs(dst + col, (col >= lo && col < hi_edge) ? __ldcs(src + col) : fill);
  }
}

namespace {
int grid_for(int64_t work_items, int dev) {
  int64_t blocks = (work_items + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count(dev)) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
}  // namespace

}  // namespace xtc

using namespace xtc;

extern "C" int xtc_cuda_relu_f32(const float* X, float* Y, int64_t n, float threshold,
                                 void* stream) {
  XTC_REQUIRE(n >= 0, "relu: negative size");
  if (n == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(X && Y, "relu: NULL operand");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (aligned16(X) && aligned16(Y))
    relu_f32_kernel<<<grid_for((n + 3) / 4, dev), 256, 0, s>>>(X, Y, n, threshold);
  else
    relu_f32_scalar_kernel<<<grid_for(n, dev), 256, 0, s>>>(X, Y, n, threshold);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_split_tf32(const float* X, float* hi, float* lo, int64_t n, void* stream) {
  XTC_REQUIRE(n >= 0, "split_tf32: negative size");
  if (n == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(X && hi && lo, "split_tf32: NULL operand");
  XTC_REQUIRE(aligned16(X) && aligned16(hi) && aligned16(lo), "split_tf32: operands must be 16-byte aligned");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  split_tf32_kernel<<<grid_for((n + 3) / 4, dev), 256, 0, static_cast<cudaStream_t>(stream)>>>(X, hi, lo, n);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_transpose_f32(const float* X, float* Y, int ndim, const int64_t* shape,
                                      const int32_t* axes, void* stream) {
  XTC_REQUIRE(ndim >= 1 && ndim <= XTC_CUDA_MAX_DIMS, "transpose: rank %d not in [1,%d]", ndim,
              XTC_CUDA_MAX_DIMS);
  XTC_REQUIRE(shape && axes, "transpose: NULL shape/axes");
  bool seen[XTC_CUDA_MAX_DIMS] = {};
  int64_t total = 1;
  for (int d = 0; d < ndim; ++d) {
    XTC_REQUIRE(axes[d] >= 0 && axes[d] < ndim && !seen[axes[d]], "transpose: axes is not a permutation");
    seen[axes[d]] = true;
    XTC_REQUIRE(shape[d] >= 0, "transpose: negative extent");
    total *= shape[d];
  }
  if (total == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(X && Y, "transpose: NULL operand");
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  // Drop unit axes, then merge input axes that stay adjacent and in order in the output.
  int64_t in_stride_full[XTC_CUDA_MAX_DIMS];
  {
    int64_t st = 1;
    for (int d = ndim - 1; d >= 0; --d) { in_stride_full[d] = st; st *= shape[d]; }
  }
  int n = 0;
  int64_t oshape[XTC_CUDA_MAX_DIMS], ostride[XTC_CUDA_MAX_DIMS];  // output dims: extent, input stride
  for (int d = 0; d < ndim; ++d) {
    const int a = axes[d];
    if (shape[a] == 1) continue;
    if (n > 0 && ostride[n - 1] == in_stride_full[a] * shape[a]) {
      // previous output dim walks the input axis just outside `a`: merge
      oshape[n - 1] *= shape[a];
      ostride[n - 1] = in_stride_full[a];
    } else {
      oshape[n] = shape[a];
      ostride[n] = in_stride_full[a];
      ++n;
    }
  }
  if (n <= 1) {  // identity permutation: plain copy
    XTC_CUDA_CHECK(cudaMemcpyAsync(Y, X, static_cast<size_t>(total) * 4, cudaMemcpyDeviceToDevice, s));
    return XTC_CUDA_OK;
  }
  int64_t out_stride[XTC_CUDA_MAX_DIMS];
  {
    int64_t st = 1;
    for (int d = n - 1; d >= 0; --d) { out_stride[d] = st; st *= oshape[d]; }
  }

  if (ostride[n - 1] == 1) {
    // innermost axis preserved: row copies
    RowCopyParams p;
    const int64_t inner = oshape[n - 1];
    bool vec = inner % 4 == 0 && aligned16(X) && aligned16(Y);
    for (int d = 0; d < n - 1; ++d) vec = vec && (ostride[d] % 4 == 0);
    const int unit = vec ? 4 : 1;
    p.ndim = n - 1;
    for (int d = 0; d < n - 1; ++d) { p.out_shape[d] = oshape[d]; p.in_stride[d] = ostride[d]; }
    p.inner = inner / unit;
    p.total = total / unit;
    if (vec)
      permute_rows_kernel<float4><<<grid_for(p.total, dev), 256, 0, s>>>(
          reinterpret_cast<const float4*>(X), reinterpret_cast<float4*>(Y), p, 4);
    else
      permute_rows_kernel<float><<<grid_for(p.total, dev), 256, 0, s>>>(X, Y, p, 1);
    XTC_CUDA_CHECK(cudaGetLastError());
    return XTC_CUDA_OK;
  }

  // General case: find the output dim that walks the input's innermost axis.
  int oc = -1;
  for (int d = 0; d < n; ++d) if (ostride[d] == 1) oc = d;
  XTC_REQUIRE(oc >= 0, "transpose: internal error (no unit-stride axis)");
  Tile2DParams p;
  p.R = oshape[n - 1];
  p.in_r_stride = ostride[n - 1];
  p.C = oshape[oc];
  p.out_c_stride = out_stride[oc];
  p.nbatch_dims = 0;
  int64_t nbatch = 1;
  for (int d = 0; d < n - 1; ++d) {
    if (d == oc) continue;
    p.batch_shape[p.nbatch_dims] = oshape[d];
    p.batch_in_stride[p.nbatch_dims] = ostride[d];
    p.batch_out_stride[p.nbatch_dims] = out_stride[d];
    nbatch *= oshape[d];
    ++p.nbatch_dims;
  }
  constexpr int TILE = 64;
  p.tiles_r = (p.R + TILE - 1) / TILE;
  p.tiles_c = (p.C + TILE - 1) / TILE;
  bool vin = aligned16(X) && p.in_r_stride % 4 == 0;
  bool vout = aligned16(Y) && p.out_c_stride % 4 == 0;
  for (int d = 0; d < p.nbatch_dims; ++d) {
    vin = vin && p.batch_in_stride[d] % 4 == 0;
    vout = vout && p.batch_out_stride[d] % 4 == 0;
  }
  p.vec_in = vin;
  p.vec_out = vout;
  // TMA path: both sides addressable by a rank-4 tensor map (16-byte aligned base and
  // pitches, at most two batch axes); anything else runs the load/store kernel below.
  if (vin && vout && p.nbatch_dims <= 2 && p.R < (1ll << 31) && p.C < (1ll << 31)) {
    const uint64_t b0 = p.nbatch_dims > 0 ? p.batch_shape[p.nbatch_dims - 1] : 1;
    const uint64_t b1 = p.nbatch_dims > 1 ? p.batch_shape[0] : 1;
    const uint64_t span = static_cast<uint64_t>(total + 3) & ~3ull;  // pitch of an absent axis
    auto bstride = [&](const int64_t* st, int which) -> uint64_t {
      if (which == 0) return p.nbatch_dims > 0 ? st[p.nbatch_dims - 1] : span;
      return p.nbatch_dims > 1 ? st[0] : span;
    };
    const uint64_t in_dims[4] = {static_cast<uint64_t>(p.C), static_cast<uint64_t>(p.R), b0, b1};
    const uint64_t in_st[3] = {static_cast<uint64_t>(p.in_r_stride), bstride(p.batch_in_stride, 0),
                               bstride(p.batch_in_stride, 1)};
    const uint64_t out_dims[4] = {static_cast<uint64_t>(p.R), static_cast<uint64_t>(p.C), b0, b1};
    const uint64_t out_st[3] = {static_cast<uint64_t>(p.out_c_stride), bstride(p.batch_out_stride, 0),
                                bstride(p.batch_out_stride, 1)};
    const uint32_t box[4] = {TT, TT, 1, 1};
    CUtensorMap tmIn, tmOut;
    int* status = device_status_word(dev);
    if (status != nullptr && make_tmap_4d_plain(&tmIn, X, in_dims, in_st, box) &&
        make_tmap_4d_plain(&tmOut, Y, out_dims, out_st, box)) {
      TmaTransposeParams tp;
      tp.tiles_c = p.tiles_c;
      tp.tiles_r = p.tiles_r;
      tp.b0 = static_cast<long long>(b0);
      tp.total = p.tiles_c * p.tiles_r * static_cast<long long>(b0 * b1);
      tp.status = status;
      static thread_local int configured_dev = -1;
      if (configured_dev != dev) {
        XTC_CUDA_CHECK(cudaFuncSetAttribute(transpose_tma_kernel,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, TT_SMEM));
        configured_dev = dev;
      }
      const long long slots = 2ll * sm_count(dev);
      const unsigned grid = static_cast<unsigned>(tp.total < slots ? tp.total : slots);
      XTC_CUDA_CHECK(launch_overlapped(transpose_tma_kernel, grid, 256, TT_SMEM, s, tmIn, tmOut, tp));
      return XTC_CUDA_OK;
    }
  }
  const int64_t blocks = nbatch * p.tiles_r * p.tiles_c;
  XTC_REQUIRE(blocks < (1ll << 31), "transpose: too many tiles");
  transpose_tile_kernel<TILE><<<static_cast<unsigned>(blocks), 256, 0, s>>>(X, Y, p);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_pad_f32(const float* X, float* Y, int ndim, const int64_t* shape,
                                const int64_t* lo, const int64_t* hi, float value, void* stream) {
  XTC_REQUIRE(ndim >= 1 && ndim <= XTC_CUDA_MAX_DIMS, "pad: rank %d not in [1,%d]", ndim,
              XTC_CUDA_MAX_DIMS);
  XTC_REQUIRE(shape && lo && hi, "pad: NULL shape/widths");
  PadParams p;
  p.ndim = ndim;
  p.value = value;
  int64_t total = 1, in_total = 1;
  for (int d = 0; d < ndim; ++d) {
    XTC_REQUIRE(shape[d] >= 0, "pad: negative extent");
    p.in_shape[d] = shape[d];
    p.out_shape[d] = shape[d] + lo[d] + hi[d];
    XTC_REQUIRE(p.out_shape[d] >= 0, "pad: axis %d cropped below zero", d);
    p.lo[d] = lo[d];
    total *= p.out_shape[d];
    in_total *= shape[d];
  }
  if (total == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(Y && (X || in_total == 0), "pad: NULL operand");
  // An axis without padding merges into its outer neighbour: [.., a, b] with b untouched is
  // [.., a*b] padded by lo_a*b and hi_a*b.  NHWC padded on H and W becomes [B, H, W*C].
  {
    int64_t hi_w[XTC_CUDA_MAX_DIMS];
    for (int d = 0; d < ndim; ++d) hi_w[d] = hi[d];
    int n = ndim;
    for (int d = n - 1; d >= 1; --d) {
      if (p.lo[d] == 0 && hi_w[d] == 0) {
        const int64_t inner = p.in_shape[d];
        p.in_shape[d - 1] *= inner;
        p.out_shape[d - 1] *= inner;
        p.lo[d - 1] *= inner;
        hi_w[d - 1] *= inner;
        for (int e = d; e < n - 1; ++e) {
          p.in_shape[e] = p.in_shape[e + 1];
          p.out_shape[e] = p.out_shape[e + 1];
          p.lo[e] = p.lo[e + 1];
          hi_w[e] = hi_w[e + 1];
        }
        --n;
      }
    }
    p.ndim = n;
    int64_t st = 1;
    for (int d = n - 1; d >= 0; --d) { p.in_stride[d] = st; st *= p.in_shape[d]; }
  }
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int last = p.ndim - 1;
  const int64_t hi_last = p.out_shape[last] - p.in_shape[last] - p.lo[last];
  const bool vec = aligned16(X) && aligned16(Y) && p.in_shape[last] % 4 == 0 && p.lo[last] % 4 == 0 &&
                   hi_last % 4 == 0 && in_total > 0;
  if (vec) {
    p.in_shape[last] /= 4;
    p.out_shape[last] /= 4;
    p.lo[last] /= 4;
    for (int d = 0; d < last; ++d) p.in_stride[d] /= 4;
  }
  const int64_t width = p.out_shape[last];
  const int64_t rows = total / (vec ? 4 : 1) / width;
  int lane_shift = 0;
  while (lane_shift < 8 && (1ll << lane_shift) < width) ++lane_shift;
  const int64_t chunk_width = (1ll << lane_shift) * 16;  // 16 accesses per thread and work item
  const int64_t chunks = (width + chunk_width - 1) / chunk_width;
  const int64_t groups = (rows * chunks + (256 >> lane_shift) - 1) / (256 >> lane_shift);
  int64_t blocks = static_cast<int64_t>(sm_count(dev)) * 8;
  if (blocks > groups) blocks = groups;
  p.total = total;
  if (vec)
    pad_kernel<float4><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        reinterpret_cast<const float4*>(X), reinterpret_cast<float4*>(Y), p, lane_shift, rows, chunks,
        chunk_width);
  else
    pad_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, s>>>(X, Y, p, lane_shift, rows, chunks,
                                                                    chunk_width);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}
