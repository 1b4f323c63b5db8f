"""Partitioning of the two multi-GPU configurations across the GPUs of one box.

One process per GPU (``torch.distributed``; NCCL over NVLink on GPUs, gloo in
the CPU tests).  The reference has no multi-GPU notion at all (its GPU runtime
is hard-wired to device 0, ``runtimes/accelerator/gpu/GPUDevice.py:95-97``), so
this module has no counterpart there; it implements the partitioning the
benchmark configurations ask for:

* row-sharded matmul (c5): rank r owns rows [r*M/g, (r+1)*M/g) of A and of C, B
  is replicated; every rank computes its block of C straight into its slot of a
  full-size C and the blocks are exchanged with an all-gather.  With
  ``chunks > 1`` the block is computed in row chunks and the exchange of chunk
  i runs on a second stream while chunk i+1 is computed.
* batch-sharded conv chain (c3): rank r owns images [r*B/g, (r+1)*B/g); no
  exchange step at all.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block [start, stop) of `total` units owned by `rank`; the first
    `total % world` ranks get one extra unit."""
    assert world >= 1 and 0 <= rank < world
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def chunk_ranges(start: int, stop: int, chunks: int) -> list[tuple[int, int]]:
    """Split [start, stop) into at most `chunks` near-equal consecutive ranges."""
    n = stop - start
    chunks = max(1, min(chunks, n)) if n > 0 else 1
    out = []
    for c in range(chunks):
        lo, hi = shard_range(n, chunks, c)
        out.append((start + lo, start + hi))
    return out


class NcclRows:
    """The NCCL communicator of the C ABI (``xtc_cuda_comm_*``, ``xtc_cuda_allgather_rows``):
    what a host without torch would use for the row exchange.  Rank 0 creates the 128-byte
    identifier; here it travels to the other ranks over the torch process group, which is
    only the out-of-band channel."""

    def __init__(self, device: Any, world: int, rank: int, group: Any = None) -> None:
        import ctypes

        import torch.distributed as dist

        from . import capi

        self._capi = capi
        self.lib = device.lib
        self.world, self.rank = world, rank
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            capi.check(self.lib.xtc_cuda_comm_unique_id(ident))
        box = [ident.raw]
        if world > 1:
            dist.broadcast_object_list(box, src=0, group=group)
        ident = ctypes.create_string_buffer(box[0], 128)
        device.activate()
        handle = ctypes.c_void_p()
        capi.check(self.lib.xtc_cuda_comm_init(ctypes.byref(handle), world, rank, ident))
        self._handle = handle

    def allgather_rows(self, ptr: int, rows_per_rank: int, row_bytes: int, lo: int = 0,
                       hi: int | None = None, stream: Any = None) -> None:
        """Rows [lo, hi) of every rank's block (block-relative) to all ranks, in place."""
        hi = rows_per_rank if hi is None else hi
        self._capi.check(self.lib.xtc_cuda_allgather_rows(
            self._handle, ptr, rows_per_rank, row_bytes, lo, hi, stream))

    def close(self) -> None:
        if self._handle:
            self._capi.check(self.lib.xtc_cuda_comm_destroy(self._handle))
            self._handle = None


@dataclass
class RowShardedMatmul:
    """C[M,N] = A[M,K] @ B[K,N] with A and C row-sharded over the process group.

    ``compute(row_lo, row_hi, stream)`` must write rows [row_lo, row_hi) of
    ``c_full`` (it is given global row numbers; the caller maps them onto its
    local A block).  ``c_full`` is a torch tensor [M, N] present on every rank.
    The exchange is torch.distributed's all-gather or, when ``comm`` is an
    ``NcclRows``, the C ABI's ``xtc_cuda_allgather_rows`` on the stream given to
    ``step`` (which must then be torch's current stream when ``chunks > 1``).
    """

    c_full: Any
    world: int
    rank: int
    compute: Callable[[int, int, Any], None]
    group: Any = None
    chunks: int = 1
    comm: Any = None

    def __post_init__(self) -> None:
        m = self.c_full.shape[0]
        assert m % self.world == 0, (
            f"row-sharded matmul needs M ({m}) divisible by the number of ranks ({self.world})")
        self.rows = m // self.world
        self.row_lo = self.rank * self.rows
        self._comm_stream = None

    def _row_bytes(self) -> int:
        return self.c_full.shape[1] * self.c_full.element_size()

    def _exchange_all(self, stream: Any = None) -> None:
        import torch.distributed as dist

        if self.world == 1:
            return
        if self.comm is not None:
            self.comm.allgather_rows(self.c_full.data_ptr(), self.rows, self._row_bytes(),
                                     stream=stream)
            return
        mine = self.c_full[self.row_lo : self.row_lo + self.rows]
        dist.all_gather_into_tensor(self.c_full, mine, group=self.group)

    def _exchange_chunk(self, lo: int, hi: int) -> list[Any]:
        """Send rows [lo, hi) of the own block to every peer and receive the peers'
        matching rows, each directly at its final place in c_full."""
        import torch.distributed as dist

        ops = []
        off_lo, off_hi = lo - self.row_lo, hi - self.row_lo
        if self.comm is not None:
            self.comm.allgather_rows(self.c_full.data_ptr(), self.rows, self._row_bytes(), off_lo,
                                     off_hi, stream=self._comm_stream.cuda_stream)
            return []
        for peer in range(self.world):
            if peer == self.rank:
                continue
            ops.append(dist.P2POp(dist.isend, self.c_full[lo:hi], peer, group=self.group))
            base = peer * self.rows
            ops.append(dist.P2POp(dist.irecv, self.c_full[base + off_lo : base + off_hi], peer,
                                  group=self.group))
        return dist.batch_isend_irecv(ops) if ops else []

    def step(self, stream: Any = None) -> None:
        """One full step: compute the own block, exchange, leave c_full complete.
        On return the work is enqueued (GPU) or done (CPU)."""
        if self.chunks <= 1 or self.world == 1:
            self.compute(self.row_lo, self.row_lo + self.rows, stream)
            self._exchange_all(stream)
            return
        import torch

        on_gpu = self.c_full.is_cuda
        pending = []
        if on_gpu:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=self.c_full.device)
            main = torch.cuda.current_stream(self.c_full.device)
        for lo, hi in chunk_ranges(self.row_lo, self.row_lo + self.rows, self.chunks):
            self.compute(lo, hi, stream)
            if on_gpu:
                ready = torch.cuda.Event()
                ready.record(main)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ready)
                    pending += self._exchange_chunk(lo, hi)
            else:
                pending += self._exchange_chunk(lo, hi)
        for req in pending:
            req.wait()
        if on_gpu:
            main.wait_stream(self._comm_stream)


class PeerStoreMatmul:
    """Row-sharded matmul with the all-gather fused into the GEMM.

    Every rank holds a full-size C allocated through the C ABI and exports it to
    the other ranks (CUDA IPC).  ``step`` launches ONE kernel per rank,
    ``xtc_cuda_gemm_f32_bcast``: its epilogue writes each finished tile of the
    rank's row block into the local C and, with plain stores over NVLink, into
    the same rows of every peer's C, so the transfer overlaps the tensor-core
    work tile by tile and needs no SMs of its own.  A tiny stream-ordered
    all-reduce afterwards is the barrier that tells each rank that all peers'
    kernels (and therefore their stores into its C) have completed.
    """

    def __init__(self, device: Any, a_ptr: int, b_ptr: int, m: int, n: int, k: int, world: int,
                 rank: int, group: Any = None, config: dict | None = None,
                 exchange: str = "peer") -> None:
        """exchange: "peer" = one 128-bit store per peer (CUDA IPC mappings of the peers' C);
        "multimem" = one multicast store per vector through an NVLink multicast object that
        every rank's C is bound to (NVLS; the buffers come from torch's symmetric-memory
        allocator), falling back to peer where the box has no multicast support when asked
        for with "multimem?"; "auto" = the faster of the two as measured on 2 and 8 B200s,
        which is peer (65536 x 8192 x 8192: 7.28 ms against 7.73 ms on 2 GPUs, 3.25 ms
        against 3.30 ms on 8: the step is bound by what every GPU has to RECEIVE, and the
        multicast delivers a rank's block to the rank itself as well).  ``self.exchange`` says
        which one runs."""
        import ctypes

        import torch
        import torch.distributed as dist

        from . import capi

        assert m % world == 0, f"M ({m}) must be divisible by the number of ranks ({world})"
        assert exchange in ("peer", "multimem", "multimem?", "auto"), exchange
        self.device, self.lib = device, device.lib
        self.world, self.rank, self.group = world, rank, group
        self.m, self.n, self.k = m, n, k
        self.rows = m // world
        self.a_ptr, self.b_ptr = int(a_ptr), int(b_ptr)
        self.cfg = capi.GemmConfig(**(config or {}))
        offset = rank * self.rows * n * 4
        self.imported: list[Any] = []
        self.mcast_block = 0
        self._symm = None
        self.exchange = "none" if world == 1 else "peer"
        if world > 1 and exchange in ("multimem", "multimem?"):
            self._symm = self._multicast_buffer(m * n, group, required=exchange == "multimem")
        if self._symm is not None:
            tensor, handle = self._symm
            self.c_local = ctypes.c_void_p(tensor.data_ptr())
            self.mcast_block = int(handle.multicast_ptr) + offset
            self.exchange = "multimem"
            extras: list[int] = []
        else:
            self.c_local = device.memory_allocate(m * n * 4)
            handle = ctypes.create_string_buffer(64)
            capi.check(self.lib.xtc_cuda_ipc_export(self.c_local, handle))
            handles: list[Any] = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            extras = []
            for r in range(world):
                if r == rank:
                    continue
                ptr = ctypes.c_void_p()
                capi.check(self.lib.xtc_cuda_ipc_import(ctypes.create_string_buffer(handles[r], 64),
                                                        ctypes.byref(ptr)))
                self.imported.append(ptr)
                extras.append(ptr.value + offset)
        self.extras = (ctypes.c_void_p * max(len(extras), 1))(*extras)
        self.n_extra = len(extras)
        self.c_block = self.c_local.value + offset
        # the workspace a plan would give this GEMM (split tail of the CTA-pair kernel), cleared once
        ws = ctypes.c_size_t(0)
        capi.check(self.lib.xtc_cuda_gemm_workspace_bytes(self.rows, n, k, 0, ctypes.byref(self.cfg),
                                                          ctypes.byref(ws)))
        self.ws_bytes = ws.value
        self.workspace = device.memory_allocate(ws.value) if ws.value else None
        if self.workspace is not None:
            device.memory_fill_zero(self.workspace, ws.value)
            device.synchronize()
        self._flag = torch.zeros(1, device="cuda")
        self._dist = dist

    def _multicast_buffer(self, numel: int, group: Any, required: bool) -> Any:
        """(tensor, handle) of a float32 buffer of `numel` elements on every rank, all bound
        to one NVLink multicast object, or None where the box cannot (every rank must take
        the same branch: the outcome is agreed on with an all-reduce)."""
        import torch
        import torch.distributed as dist

        pair, reason = None, ""
        try:
            import torch.distributed._symmetric_memory as symm_mem

            pg = group if group is not None else dist.group.WORLD
            tensor = symm_mem.empty((numel,), dtype=torch.float32,
                                    device=torch.device("cuda", self.device.ordinal))
            handle = symm_mem.rendezvous(tensor, pg)
            if int(getattr(handle, "multicast_ptr", 0) or 0) != 0:
                pair = (tensor, handle)
            else:
                reason = "the symmetric-memory handle has no multicast address"
        except Exception as e:  # allocator or driver without multicast support
            reason = f"{type(e).__name__}: {e}"
        ok = torch.tensor([1.0 if pair is not None else 0.0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() != 1.0:
            if required:
                raise RuntimeError(f"multimem exchange unavailable on rank {self.rank}: {reason or 'a peer could not'}")
            return None
        return pair

    def _on_stream(self, stream: int | None) -> Any:
        """Context that makes `stream` (a raw cudaStream_t; None or 0 = the legacy default
        stream) torch's current stream, so that a collective issued inside it is ordered
        after the kernels this object launched on that stream."""
        import torch

        if not stream:
            return torch.cuda.stream(torch.cuda.default_stream())
        return torch.cuda.stream(torch.cuda.ExternalStream(int(stream)))

    def step(self, stream: int | None = None) -> None:
        from . import capi

        if self.mcast_block:
            rc = self.lib.xtc_cuda_gemm_f32_mcast(
                self.a_ptr, self.b_ptr, self.c_block, self.mcast_block, self.rows, self.n, self.k,
                self.k, self.n, self.n, 0, 0.0, ctypes_byref(self.cfg), self.workspace,
                self.ws_bytes, stream)
        else:
            rc = self.lib.xtc_cuda_gemm_f32_bcast(
                self.a_ptr, self.b_ptr, self.c_block, self.extras, self.n_extra, self.rows, self.n,
                self.k, self.k, self.n, self.n, 0, 0.0, ctypes_byref(self.cfg), self.workspace,
                self.ws_bytes, stream)
        if rc:
            capi.check(rc)
        if self.world > 1:
            # the barrier that says "every peer's stores into my C have landed": it must
            # follow the GEMM on the GEMM's own stream, whatever torch's current stream is
            with self._on_stream(stream):
                self._dist.all_reduce(self._flag, group=self.group)

    def drain(self) -> None:
        """The exchange is part of the step's kernel: nothing runs behind the step's stream."""

    def host_loop(self) -> "ShardedHostLoop":
        """Overlapped executor of this step on host batches (see ShardedHostLoop)."""
        return ShardedHostLoop(self)

    def result(self) -> Any:
        """The full C of this rank as a NumPy array (synchronises)."""
        import numpy as np

        out = np.empty((self.m, self.n), np.float32)
        self.device.memory_copy_from(self.c_local, out, out.nbytes)
        return out

    def close(self) -> None:
        if self.world > 1:
            # nobody may still be storing into a C that is about to be freed: every kernel of
            # every stream of this device first, then all ranks meet
            self.device.synchronize()
            self._dist.barrier(group=self.group)
        for ptr in self.imported:
            self.lib.xtc_cuda_ipc_release(ptr)
        self.imported = []
        if self.world > 1:
            self._dist.barrier(group=self.group)  # nobody frees a C that a peer still has mapped
        if self._symm is not None:
            # drop the multicast binding while every rank is still alive (all ranks are past
            # the barrier above, none has exited)
            self._symm = None
            self.c_local = None
            self.mcast_block = 0
            import torch

            torch.cuda.synchronize()
            self._dist.barrier(group=self.group)
        if self.c_local is not None:
            self.device.memory_free(self.c_local)
            self.c_local = None
        if self.workspace is not None:
            self.device.memory_free(self.workspace)
            self.workspace = None


class PipelinedPeerMatmul:
    """Row-sharded matmul whose exchange runs one step behind the product.

    Where the exchange takes longer than the product (65536 x 8192 x 8192 on 8 GPUs: every
    GPU computes for 1.5 ms and has to receive 1.88 GB), fusing the two into one kernel cannot
    beat the link, and the fused kernel's stores reach 590 - 665 GB/s where a peer copy by the
    copy engines reaches 770.  Here a step is the plain GEMM into this rank's rows of one of
    TWO full-size C buffers; the rows then travel to every peer's copy of that buffer with one
    peer-to-peer ``xtc_cuda_memcpy_d2d`` per peer (CUDA IPC mappings, copy engines, no SM) on a
    second stream while the next step's GEMM runs, in a rotation (rank r sends to r+1, r+2,
    ...) that has every GPU receive from one peer at a time.  ``xtc_cuda_peer_barrier`` after
    the copies (one warp that writes a flag into every peer's memory and waits for theirs) says
    "every peer's rows of this step have landed"; a library collective in that place wants SM
    resources of its own and delays the next GEMM launch by 0.3 - 0.6 ms.

    Throughput per step is then max(product, exchange) instead of their fused sum;
    ``result_of(step)`` is complete after ``wait()`` (or, stream-ordered, after the
    barrier of that step on the exchange stream).  Step i + 2 reuses the buffer of step i:
    a consumer must have read a step's C before submitting the step after next.
    """

    def __init__(self, device: Any, a_ptr: int, b_ptr: int, m: int, n: int, k: int, world: int,
                 rank: int, group: Any = None, config: dict | None = None) -> None:
        import ctypes

        import torch.distributed as dist

        from . import capi

        assert m % world == 0, f"M ({m}) must be divisible by the number of ranks ({world})"
        assert 1 <= world <= 8, f"the barrier's flag array has 8 slots: {world} ranks do not fit"
        self.device, self.lib = device, device.lib
        self.world, self.rank, self.group = world, rank, group
        self.m, self.n, self.k = m, n, k
        self.rows = m // world
        self.a_ptr, self.b_ptr = int(a_ptr), int(b_ptr)
        self.cfg = capi.GemmConfig(**(config or {}))
        self.exchange = "none" if world == 1 else "pipelined peer copies"
        self.offset = rank * self.rows * n * 4
        self.block_bytes = self.rows * n * 4
        self.buffers = [device.memory_allocate(m * n * 4) for _ in range(2)]
        self.imported: list[Any] = []
        # peers[b][j] = buffer b of rank (rank + 1 + j) % world, mapped here
        self.peers: list[list[int]] = [[], []]
        for b in range(2):
            handle = ctypes.create_string_buffer(64)
            capi.check(self.lib.xtc_cuda_ipc_export(self.buffers[b], handle))
            handles: list[Any] = [None] * world
            if world > 1:
                dist.all_gather_object(handles, handle.raw, group=group)
            for j in range(1, world):
                r = (rank + j) % world
                ptr = ctypes.c_void_p()
                capi.check(self.lib.xtc_cuda_ipc_import(ctypes.create_string_buffer(handles[r], 64),
                                                        ctypes.byref(ptr)))
                self.imported.append(ptr)
                self.peers[b].append(ptr.value)
        # the barrier's flags: 8 ints per rank, each rank's array mapped by all the others
        self.flags = device.memory_allocate(256)
        device.memory_fill_zero(self.flags, 256)
        device.synchronize()
        handle = ctypes.create_string_buffer(64)
        capi.check(self.lib.xtc_cuda_ipc_export(self.flags, handle))
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        peer_flags, peer_ranks = [], []
        for j in range(1, world):
            r = (rank + j) % world
            ptr = ctypes.c_void_p()
            capi.check(self.lib.xtc_cuda_ipc_import(ctypes.create_string_buffer(handles[r], 64),
                                                    ctypes.byref(ptr)))
            self.imported.append(ptr)
            peer_flags.append(ptr.value)
            peer_ranks.append(r)
        self.peer_flags = (ctypes.c_void_p * max(world - 1, 1))(*peer_flags)
        self.peer_ranks = (ctypes.c_int * max(world - 1, 1))(*peer_ranks)
        ws = ctypes.c_size_t(0)
        capi.check(self.lib.xtc_cuda_gemm_workspace_bytes(self.rows, n, k, 0, ctypes.byref(self.cfg),
                                                          ctypes.byref(ws)))
        self.ws_bytes = ws.value
        self.workspace = device.memory_allocate(ws.value) if ws.value else None
        if self.workspace is not None:
            device.memory_fill_zero(self.workspace, ws.value)
            device.synchronize()
        if world > 1:
            dist.barrier(group=group)  # every rank's flags are zero and mapped before the first step

        def make(fn: Any) -> Any:
            h = ctypes.c_void_p()
            capi.check(fn(ctypes.byref(h)))
            return h

        self.s_copy = make(self.lib.xtc_cuda_stream_create)
        self.ev_gemm = [make(self.lib.xtc_cuda_event_create) for _ in range(2)]
        self.ev_sent = [make(self.lib.xtc_cuda_event_create) for _ in range(2)]
        self.steps = 0
        self._dist, self._check = dist, capi.check

    def step(self, stream: int | None = None) -> None:
        """Enqueue one step: the GEMM on `stream`, its exchange on the copy stream behind it."""
        lib, ck = self.lib, self._check
        b = self.steps & 1
        if self.steps >= 2:
            # the rows of step i - 2 have left this buffer
            ck(lib.xtc_cuda_stream_wait_event(stream, self.ev_sent[b]))
        rc = lib.xtc_cuda_gemm_f32(self.a_ptr, self.b_ptr, self.buffers[b].value + self.offset, self.rows,
                                   self.n, self.k, self.k, self.n, self.n, 0, 0.0, ctypes_byref(self.cfg),
                                   self.workspace, self.ws_bytes, stream)
        if rc:
            ck(rc)
        if self.world > 1:
            ck(lib.xtc_cuda_event_record(self.ev_gemm[b], stream))
            ck(lib.xtc_cuda_stream_wait_event(self.s_copy, self.ev_gemm[b]))
            src = self.buffers[b].value + self.offset
            for peer in self.peers[b]:
                ck(lib.xtc_cuda_memcpy_d2d(peer + self.offset, src, self.block_bytes, self.s_copy))
            ck(lib.xtc_cuda_peer_barrier(self.flags, self.peer_flags, self.peer_ranks, self.world - 1,
                                         self.rank, self.steps + 1, self.s_copy))
        ck(lib.xtc_cuda_event_record(self.ev_sent[b], self.s_copy if self.world > 1 else stream))
        self.steps += 1

    @property
    def c_local(self) -> Any:
        """The full-size C of the step enqueued last."""
        return self.buffers[(self.steps - 1) & 1 if self.steps else 0]

    @property
    def c_block(self) -> int:
        """This rank's rows in the C of the step enqueued last."""
        return self.c_local.value + self.offset

    def drain(self) -> None:
        """Returns when the exchange of every step enqueued so far has completed here."""
        self._check(self.lib.xtc_cuda_stream_synchronize(self.s_copy))

    def host_loop(self) -> "ShardedHostLoop":
        """Overlapped executor of this step on host batches (see ShardedHostLoop)."""
        return ShardedHostLoop(self)

    def result(self) -> Any:
        """The full C of the step enqueued last as a NumPy array (synchronises)."""
        import numpy as np

        self.device.synchronize()
        out = np.empty((self.m, self.n), np.float32)
        self.device.memory_copy_from(self.c_local, out, out.nbytes)
        return out

    def close(self) -> None:
        if self.s_copy is None:
            return
        self.device.synchronize()
        if self.world > 1:
            self._dist.barrier(group=self.group)
        for ptr in self.imported:
            self.lib.xtc_cuda_ipc_release(ptr)
        self.imported = []
        if self.world > 1:
            self._dist.barrier(group=self.group)  # nobody frees memory that a peer still has mapped
        for buf in self.buffers + [self.flags]:
            self.device.memory_free(buf)
        self.buffers = []
        if self.workspace is not None:
            self.device.memory_free(self.workspace)
            self.workspace = None
        for ev in self.ev_gemm + self.ev_sent:
            self.lib.xtc_cuda_event_destroy(ev)
        self.lib.xtc_cuda_stream_destroy(self.s_copy)
        self.s_copy = None


class ShardedHostLoop:
    """Runs a PeerStoreMatmul (or PipelinedPeerMatmul) step on a sequence of host batches.

    ``submit(host_a, host_c)`` copies this rank's block of A in from host memory, runs the
    fused GEMM + exchange, and copies this rank's block of C back out; the copy-in of step
    i+1 and the copy-out of step i run side by side on streams of their own (the host link
    is full duplex) while the step itself occupies a third.  One device A block and one C
    are shared by all steps, so a step's GEMM waits for the previous step's copy-out and a
    copy-in waits for the previous GEMM.  ``wait()`` returns when every submitted step has
    delivered, and raises if a kernel reported a bounded-wait timeout.  Host arrays should
    be page-locked (``xtc_cuda_host_alloc``) for the copies to overlap.  Every rank must
    submit the same number of steps (each step ends in a collective barrier).
    """

    def __init__(self, op: "PeerStoreMatmul") -> None:
        import ctypes

        from . import capi

        self.op, self.lib = op, op.lib
        self._check = capi.check

        def make(fn: Any) -> Any:
            h = ctypes.c_void_p()
            capi.check(fn(ctypes.byref(h)))
            return h

        self.s_in, self.s_run, self.s_out = (make(self.lib.xtc_cuda_stream_create) for _ in range(3))
        self.ev_in, self.ev_run, self.ev_out = (make(self.lib.xtc_cuda_event_create) for _ in range(3))
        self.submitted = 0
        self.a_bytes = op.rows * op.k * 4
        self.c_bytes = op.rows * op.n * 4

    def submit(self, host_a: int, host_c: int) -> None:
        """host_a / host_c: addresses of this rank's [rows, K] block of A and [rows, N] block of C."""
        lib, ck = self.lib, self._check
        if self.submitted:
            ck(lib.xtc_cuda_stream_wait_event(self.s_in, self.ev_run))   # A is free again
        ck(lib.xtc_cuda_memcpy_h2d(self.op.a_ptr, host_a, self.a_bytes, self.s_in))
        ck(lib.xtc_cuda_event_record(self.ev_in, self.s_in))
        ck(lib.xtc_cuda_stream_wait_event(self.s_run, self.ev_in))
        if self.submitted:
            ck(lib.xtc_cuda_stream_wait_event(self.s_run, self.ev_out))  # C block has been read out
        self.op.step(self.s_run.value)
        ck(lib.xtc_cuda_event_record(self.ev_run, self.s_run))
        ck(lib.xtc_cuda_stream_wait_event(self.s_out, self.ev_run))
        ck(lib.xtc_cuda_memcpy_d2h(host_c, self.op.c_block, self.c_bytes, self.s_out))
        ck(lib.xtc_cuda_event_record(self.ev_out, self.s_out))
        self.submitted += 1

    def wait(self) -> None:
        from . import capi

        if self.submitted:
            self._check(self.lib.xtc_cuda_event_synchronize(self.ev_out))
        self.op.drain()
        if self.op.device.status() != 0:
            raise capi.XtcCudaError(capi.ERR_DEVICE_TIMEOUT, "a kernel's bounded wait gave up")

    def close(self) -> None:
        if self.s_in is None:
            return
        self.op.device.synchronize()
        for ev in (self.ev_in, self.ev_run, self.ev_out):
            self.lib.xtc_cuda_event_destroy(ev)
        for st in (self.s_in, self.s_run, self.s_out):
            self.lib.xtc_cuda_stream_destroy(st)
        self.s_in = self.s_run = self.s_out = None


def ctypes_byref(obj: Any) -> Any:
    import ctypes

    return ctypes.byref(obj)


@dataclass
class BatchSharded:
    """A graph whose leading (batch) dimension is split over the ranks; every rank
    runs the same plan on its images and nothing is exchanged."""

    total_batch: int
    world: int
    rank: int

    def __post_init__(self) -> None:
        self.lo, self.hi = shard_range(self.total_batch, self.world, self.rank)

    @property
    def local_batch(self) -> int:
        return self.hi - self.lo
