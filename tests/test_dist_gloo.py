"""The multi-GPU partitioning logic on CPU: two gloo ranks as child processes.

The per-rank compute is the oracle's matmul / conv (a stand-in for the CUDA
plan, which cannot run here); what is checked is the part that is the same on
GPUs: who owns which rows or images, where blocks land in the full result, the
all-gather and the chunked exchange, and that every rank ends with the full
result of the unsharded computation.
"""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from oracle import xtc_oracle as xo  # noqa: E402
from xtc_b200.dist import BatchSharded, RowShardedMatmul, chunk_ranges, shard_range  # noqa: E402


def test_shard_ranges_cover_without_overlap():
    for total, world in [(65536, 8), (32, 8), (10, 4), (3, 4), (7, 1)]:
        spans = [shard_range(total, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1
    assert chunk_ranges(100, 110, 4) == [(100, 103), (103, 106), (106, 108), (108, 110)]
    assert chunk_ranges(5, 6, 8) == [(5, 6)]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, chunks: int, out_dir: str) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- row-sharded matmul (c5 at 1/128 scale) --------------------------------
        a, b = xo.config_inputs("c5", 128)  # [512, 64] @ [64, 64]
        m = a.shape[0]
        c_full = torch.zeros(m, b.shape[1])
        rows = m // world
        a_blk = a[rank * rows:(rank + 1) * rows]  # the only rows of A this rank holds
        calls = []

        def compute(lo, hi, _stream):
            calls.append((lo, hi))
            local = a_blk[lo - rank * rows: hi - rank * rows]
            c_full[lo:hi] = torch.from_numpy(xo.matmul(local, b))

        op = RowShardedMatmul(c_full, world, rank, compute, chunks=chunks)
        op.step()
        ref = xo.matmul(a, b)
        assert np.array_equal(c_full.numpy(), ref), "every rank must hold the full product"
        assert calls[0][0] == rank * rows and calls[-1][1] == (rank + 1) * rows
        assert len(calls) == max(chunks, 1)
        op.step()  # a second step reuses the buffers
        assert np.array_equal(c_full.numpy(), ref)

        # ---- batch-sharded conv chain (c3 with 4 images) -----------------------------
        x, w = xo.config_inputs("c3", 8)
        sh = BatchSharded(x.shape[0], world, rank)
        y_local = xo.config_forward("c3", [x[sh.lo:sh.hi], w])
        gathered = [torch.zeros_like(torch.from_numpy(y_local)) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(y_local))  # validation only: c3 needs no collective
        full = np.concatenate([g.numpy() for g in gathered])
        assert np.array_equal(full, xo.config_forward("c3", [x, w]))
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 4])
def test_two_ranks_gloo(tmp_path, chunks):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), chunks, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_a_rank_that_raises_is_reported(tmp_path):
    """Host-side failure detection: a rank that dies before joining makes spawn raise."""
    def run():
        mp.spawn(_failing_worker, args=(2, _free_port()), nprocs=2, join=True)
    with pytest.raises(Exception):
        run()


def _failing_worker(rank: int, world: int, port: int) -> None:
    if rank == 1:
        raise RuntimeError("rank 1 fails before any collective")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
