// NCCL row exchange behind the C ABI: the library all-gather of a row-sharded
// matmul for hosts that do not want the fused peer-store epilogue
// (xtc_cuda_gemm_f32_bcast).  One process per GPU; the communicator is built
// from a 128-byte identifier that rank 0 creates and the host passes to the
// other ranks by whatever channel it has.
//
// NCCL is resolved with dlopen at the first use, so the kernel library carries
// no link-time dependency on it and loads on a machine that has none; in a
// process that already holds an NCCL (PyTorch's) the same copy is used.
#include <dlfcn.h>

#include <mutex>

#include "common.cuh"

namespace {

// The handful of NCCL declarations this file needs, as its public header gives
// them (nccl.h: ncclUniqueId is 128 opaque bytes, results and data types are
// plain enums, ncclSuccess == 0, ncclUint8 == 1).
struct nccl_unique_id {
  char internal[128];
};
typedef void* nccl_comm_t;
constexpr int NCCL_SUCCESS = 0;
constexpr int NCCL_UINT8 = 1;

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(nccl_unique_id*) = nullptr;
  int (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
  int (*CommDestroy)(nccl_comm_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  const char* why = nullptr;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  if (!g_nccl.handle) {
    g_nccl.why = "libnccl.so.2 cannot be loaded";
    return;
  }
  struct {
    const char* name;
    void** slot;
  } syms[] = {
      {"ncclGetUniqueId", (void**)&g_nccl.GetUniqueId},
      {"ncclCommInitRank", (void**)&g_nccl.CommInitRank},
      {"ncclCommDestroy", (void**)&g_nccl.CommDestroy},
      {"ncclAllGather", (void**)&g_nccl.AllGather},
      {"ncclBroadcast", (void**)&g_nccl.Broadcast},
      {"ncclGroupStart", (void**)&g_nccl.GroupStart},
      {"ncclGroupEnd", (void**)&g_nccl.GroupEnd},
      {"ncclGetErrorString", (void**)&g_nccl.GetErrorString},
  };
  for (auto& s : syms) {
    *s.slot = dlsym(g_nccl.handle, s.name);
    if (!*s.slot) {
      g_nccl.why = "the loaded NCCL lacks a symbol this library needs";
      return;
    }
  }
}

int nccl_ready(const char* who) {
  std::call_once(g_nccl_once, load_nccl);
  if (g_nccl.why) {
    xtc::set_error("%s: %s", who, g_nccl.why);
    return XTC_CUDA_ERR_UNSUPPORTED;
  }
  return XTC_CUDA_OK;
}

#define XTC_NCCL_CHECK(who, expr)                                                   \
  do {                                                                              \
    int _r = (expr);                                                                \
    if (_r != NCCL_SUCCESS) {                                                       \
      ::xtc::set_error("%s: %s failed: %s", who, #expr, g_nccl.GetErrorString(_r)); \
      return XTC_CUDA_ERR_RUNTIME;                                                  \
    }                                                                               \
  } while (0)

}  // namespace

struct xtc_cuda_comm {
  nccl_comm_t comm = nullptr;
  int world = 0;
  int rank = 0;
};

extern "C" int xtc_cuda_comm_unique_id(void* id128) {
  XTC_REQUIRE(id128, "comm_unique_id: NULL argument");
  if (int rc = nccl_ready("comm_unique_id")) return rc;
  nccl_unique_id id;
  XTC_NCCL_CHECK("comm_unique_id", g_nccl.GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_comm_init(xtc_cuda_comm** comm, int world, int rank, const void* id128) {
  XTC_REQUIRE(comm && id128, "comm_init: NULL argument");
  *comm = nullptr;
  XTC_REQUIRE(world >= 1 && rank >= 0 && rank < world, "comm_init: rank %d of %d", rank, world);
  if (int rc = nccl_ready("comm_init")) return rc;
  nccl_unique_id id;
  memcpy(&id, id128, sizeof(id));
  auto* c = new xtc_cuda_comm;
  c->world = world;
  c->rank = rank;
  int r = g_nccl.CommInitRank(&c->comm, world, id, rank);
  if (r != NCCL_SUCCESS) {
    xtc::set_error("comm_init: ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
    delete c;
    return XTC_CUDA_ERR_RUNTIME;
  }
  *comm = c;
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_allgather_rows(xtc_cuda_comm* comm, void* c, int64_t rows_per_rank,
                                       int64_t row_bytes, int64_t row_lo, int64_t row_hi,
                                       void* stream) {
  XTC_REQUIRE(comm && comm->comm, "allgather_rows: NULL communicator");
  XTC_REQUIRE(c, "allgather_rows: NULL buffer");
  XTC_REQUIRE(rows_per_rank > 0 && row_bytes > 0, "allgather_rows: %lld rows of %lld bytes",
              (long long)rows_per_rank, (long long)row_bytes);
  XTC_REQUIRE(0 <= row_lo && row_lo <= row_hi && row_hi <= rows_per_rank,
              "allgather_rows: rows [%lld, %lld) of a block of %lld", (long long)row_lo,
              (long long)row_hi, (long long)rows_per_rank);
  const int64_t limit = INT64_MAX / row_bytes / comm->world;
  XTC_REQUIRE(rows_per_rank <= limit, "allgather_rows: the gathered buffer overflows 63 bits");
  if (row_lo == row_hi || comm->world == 1) return XTC_CUDA_OK;
  if (int rc = nccl_ready("allgather_rows")) return rc;
  auto s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(c);
  const size_t block = size_t(rows_per_rank) * size_t(row_bytes);
  if (row_lo == 0 && row_hi == rows_per_rank) {
    // the whole block: NCCL's in-place form (send = recv + rank * count)
    XTC_NCCL_CHECK("allgather_rows", g_nccl.AllGather(base + size_t(comm->rank) * block, base,
                                                      block, NCCL_UINT8, comm->comm, s));
    return XTC_CUDA_OK;
  }
  // a row range of every block: one in-place broadcast per owner, as one group
  const size_t off = size_t(row_lo) * size_t(row_bytes);
  const size_t bytes = size_t(row_hi - row_lo) * size_t(row_bytes);
  XTC_NCCL_CHECK("allgather_rows", g_nccl.GroupStart());
  int first_error = NCCL_SUCCESS;
  for (int r = 0; r < comm->world; ++r) {
    char* p = base + size_t(r) * block + off;
    int e = g_nccl.Broadcast(p, p, bytes, NCCL_UINT8, r, comm->comm, s);
    if (e != NCCL_SUCCESS && first_error == NCCL_SUCCESS) first_error = e;
  }
  int end = g_nccl.GroupEnd();
  if (first_error == NCCL_SUCCESS) first_error = end;
  if (first_error != NCCL_SUCCESS) {
    xtc::set_error("allgather_rows: ncclBroadcast group failed: %s",
                   g_nccl.GetErrorString(first_error));
    return XTC_CUDA_ERR_RUNTIME;
  }
  return XTC_CUDA_OK;
}

// ---------------------------------------------------------------------------
// A barrier between the GPUs of a box that needs no SM to itself
// ---------------------------------------------------------------------------
// One warp: lane j stores `epoch` into slot `my_rank` of peer j's flag array (a mapping of the
// peer's memory, system-scope release: everything this stream did before, peer copies
// included, is visible first) and then waits, for at most about 2 s, until slot peer_rank[j]
// of the local array has reached `epoch`.  A collective of a library would do, but its kernel
// wants SM resources of its own and, launched beside a persistent GEMM that holds every SM,
// delays that GEMM's next launch (measured: 0.3 - 0.6 ms per step on 2 GPUs); this warp fits
// beside a GEMM CTA.  The kernels that wait for one another run on different GPUs.
namespace xtc {
struct PeerBarrierArgs {
  int* peer_flags[7];
  int peer_rank[7];
};
__global__ void peer_barrier_kernel(int* local_flags, PeerBarrierArgs args, int n_peers, int my_rank,
                                    int epoch, int* status) {
  const int j = threadIdx.x;
  if (j >= n_peers) return;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(args.peer_flags[j] + my_rank), "r"(epoch)
               : "memory");
  const int* mine = local_flags + args.peer_rank[j];
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (seen - epoch >= 0) return;
    if ((it & 0xff) == 0xff) {
      const uint64_t now = dev::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 2000000000ull) {
        atomicCAS(status, 0, dev::STATUS_WAIT_TIMEOUT_ACC);
        return;
      }
    }
  }
}
}  // namespace xtc

extern "C" int xtc_cuda_peer_barrier(int* local_flags, int* const* peer_flags, const int* peer_ranks,
                                     int n_peers, int my_rank, int epoch, void* stream) {
  XTC_REQUIRE(n_peers >= 0 && n_peers <= 7, "peer_barrier: %d peers (at most 7)", n_peers);
  if (n_peers == 0) return XTC_CUDA_OK;
  XTC_REQUIRE(local_flags && peer_flags && peer_ranks, "peer_barrier: NULL argument");
  XTC_REQUIRE(my_rank >= 0 && my_rank < 8, "peer_barrier: rank %d not in [0, 8)", my_rank);
  xtc::PeerBarrierArgs args;
  memset(&args, 0, sizeof(args));
  for (int j = 0; j < n_peers; ++j) {
    XTC_REQUIRE(peer_flags[j] != nullptr && peer_ranks[j] >= 0 && peer_ranks[j] < 8 &&
                    peer_ranks[j] != my_rank,
                "peer_barrier: peer %d is NULL or has a rank outside [0, 8)", j);
    args.peer_flags[j] = peer_flags[j];
    args.peer_rank[j] = peer_ranks[j];
  }
  int dev = 0;
  XTC_CUDA_CHECK(cudaGetDevice(&dev));
  int* word = xtc::device_status_word(dev);
  XTC_REQUIRE(word != nullptr, "peer_barrier: device status word unavailable");
  xtc::peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(local_flags, args, n_peers,
                                                                             my_rank, epoch, word);
  XTC_CUDA_CHECK(cudaGetLastError());
  return XTC_CUDA_OK;
}

extern "C" int xtc_cuda_comm_destroy(xtc_cuda_comm* comm) {
  if (!comm) return XTC_CUDA_OK;
  int r = comm->comm ? g_nccl.CommDestroy(comm->comm) : NCCL_SUCCESS;
  delete comm;
  if (r != NCCL_SUCCESS) {
    xtc::set_error("comm_destroy: ncclCommDestroy failed: %s", g_nccl.GetErrorString(r));
    return XTC_CUDA_ERR_RUNTIME;
  }
  return XTC_CUDA_OK;
}
