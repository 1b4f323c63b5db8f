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


@dataclass
class RowShardedMatmul:
    """C[M,N] = A[M,K] @ B[K,N] with A and C row-sharded over the process group.

    ``compute(row_lo, row_hi, stream)`` must write rows [row_lo, row_hi) of
    ``c_full`` (it is given global row numbers; the caller maps them onto its
    local A block).  ``c_full`` is a torch tensor [M, N] present on every rank.
    """

    c_full: Any
    world: int
    rank: int
    compute: Callable[[int, int, Any], None]
    group: Any = None
    chunks: int = 1

    def __post_init__(self) -> None:
        m = self.c_full.shape[0]
        assert m % self.world == 0, (
            f"row-sharded matmul needs M ({m}) divisible by the number of ranks ({self.world})")
        self.rows = m // self.world
        self.row_lo = self.rank * self.rows
        self._comm_stream = None

    def _exchange_all(self) -> None:
        import torch.distributed as dist

        if self.world == 1:
            return
        mine = self.c_full[self.row_lo : self.row_lo + self.rows]
        dist.all_gather_into_tensor(self.c_full, mine, group=self.group)

    def _exchange_chunk(self, lo: int, hi: int) -> list[Any]:
        """Send rows [lo, hi) of the own block to every peer and receive the peers'
        matching rows, each directly at its final place in c_full."""
        import torch.distributed as dist

        ops = []
        off_lo, off_hi = lo - self.row_lo, hi - self.row_lo
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
            self._exchange_all()
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
