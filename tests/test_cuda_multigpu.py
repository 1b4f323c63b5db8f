"""Row-sharded matmul on two GPUs: NCCL all-gather and the fused peer-store GEMM.

Skipped on boxes with fewer than two GPUs.  Two child processes (one per GPU)
run the same code `bench.py --gpus N` runs; every rank must end with the full
product, equal bit for bit to what one GPU computes alone and within the TF32
tolerance of the float64 oracle.
"""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu

TF32_TOL = 1e-2


def _gpu_count() -> int:
    try:
        from xtc_b200.runtimes.cuda import CudaDevice

        return CudaDevice.count()
    except Exception:
        return 0


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist

    from oracle import xtc_oracle as xo
    from xtc_b200 import capi, configs
    from xtc_b200.backends.cuda.module import PlanHandle
    from xtc_b200.dist import NcclRows, PeerStoreMatmul, PipelinedPeerMatmul, RowShardedMatmul, chunk_ranges
    from xtc_b200.runtimes.cuda import CudaDevice

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dev = CudaDevice(rank)
    dev.activate()
    try:
        a, b = xo.config_inputs("c5", 16)  # A [4096, 512], B [512, 512]
        m, k = a.shape
        n = b.shape[1]
        rows = m // world
        y64 = a.astype(np.float64) @ b.astype(np.float64)
        a_blk = torch.from_numpy(a[rank * rows:(rank + 1) * rows]).cuda()
        b_dev = torch.from_numpy(b).cuda()
        stream = torch.cuda.current_stream().cuda_stream

        # what one GPU computes alone, for the bit-for-bit comparison
        a_all = torch.from_numpy(a).cuda()
        single = torch.empty(m, n, device="cuda")
        full = PlanHandle(configs.compile_config(configs.build("c5", rows=m, scale=16)).plan, dev)
        full.run([a_all.data_ptr(), b_dev.data_ptr(), single.data_ptr()], stream)
        torch.cuda.synchronize()
        single = single.cpu().numpy()
        assert xo.rel_err(single, y64) <= TF32_TOL

        module = configs.compile_config(configs.build("c5", rows=rows, scale=16))
        handle = PlanHandle(module.plan, dev)

        # ---- NCCL all-gather -----------------------------------------------------
        c_full = torch.zeros(m, n, device="cuda")

        def compute(lo, hi, _s):
            assert (lo, hi) == (rank * rows, (rank + 1) * rows)
            handle.run([a_blk.data_ptr(), b_dev.data_ptr(), c_full[lo:hi].data_ptr()], stream)

        RowShardedMatmul(c_full, world, rank, compute).step(stream)
        torch.cuda.synchronize()
        assert np.array_equal(c_full.cpu().numpy(), single)

        # ---- the same exchange through the C ABI's own NCCL communicator ----------------
        comm = NcclRows(dev, world, rank)
        c_full.zero_()
        RowShardedMatmul(c_full, world, rank, compute, comm=comm).step(stream)
        torch.cuda.synchronize()
        assert np.array_equal(c_full.cpu().numpy(), single)
        # ... and in three row ranges of every block (what a chunked overlap issues)
        c_full.zero_()
        compute(rank * rows, (rank + 1) * rows, stream)
        for lo, hi in chunk_ranges(0, rows, 3):
            comm.allgather_rows(c_full.data_ptr(), rows, n * 4, lo, hi, stream)
        torch.cuda.synchronize()
        assert np.array_equal(c_full.cpu().numpy(), single)
        with pytest.raises(RuntimeError, match="rows"):
            comm.allgather_rows(c_full.data_ptr(), rows, n * 4, 0, rows + 1, stream)
        dist.barrier()
        comm.close()

        # ---- fused peer stores -----------------------------------------------------
        pair_cfg = dict(module.plan.steps[-1].config)
        variants = [
            pair_cfg,                                     # CTA pairs, peers written by copier warps
            dict(pair_cfg, variant=1),                    # CTA pairs, peers written by the epilogue
            dict(tile_m=128, tile_n=128, tile_k=32, epilogue=2),  # one CTA per tile
        ]
        for cfg in variants:
            op = PeerStoreMatmul(dev, a_blk.data_ptr(), b_dev.data_ptr(), m, n, k, world, rank,
                                 config=cfg)
            for _ in range(2):
                op.step(stream)
            torch.cuda.synchronize()
            dist.barrier()
            got = op.result()
            if cfg.get("tile_m") == pair_cfg.get("tile_m"):
                assert np.array_equal(got, single), "every rank must hold the full product"
            else:
                assert xo.rel_err(got, y64) <= TF32_TOL
            op.close()
            assert dev.status() == 0
        # ---- the same step from host batches, on streams that are not torch's current one ----
        op = PeerStoreMatmul(dev, a_blk.data_ptr(), b_dev.data_ptr(), m, n, k, world, rank,
                             config=pair_cfg)
        loop = op.host_loop()
        host_a = torch.from_numpy(a[rank * rows:(rank + 1) * rows].copy()).pin_memory()
        host_c = torch.full((rows, n), float("nan")).pin_memory()
        a_blk.zero_()  # the loop must bring the block in itself
        for _ in range(3):
            loop.submit(host_a.data_ptr(), host_c.data_ptr())
        loop.wait()
        dist.barrier()
        assert np.array_equal(host_c.numpy(), single[rank * rows:(rank + 1) * rows])
        assert np.array_equal(op.result(), single), "peers' blocks arrived although no stream was current"
        loop.close()
        op.close()
        assert dev.status() == 0
        # ---- the exchange one step behind the product: peer copies on a second stream --------
        op = PipelinedPeerMatmul(dev, a_blk.data_ptr(), b_dev.data_ptr(), m, n, k, world, rank, config=pair_cfg)
        for _ in range(5):
            op.step(stream)
        assert np.array_equal(op.result(), single), "the last step's C, complete on every rank"
        dist.barrier()
        # every step's own data: A is scaled by a power of two before each step (exact), the
        # steps are enqueued back to back, and the two buffers still held must carry the last
        # two steps' products on every rank (a flag that overtook its rows would show here)
        scales = [2.0, 0.5, 4.0, 0.25, 8.0, 1.0]
        a_keep = a_blk.clone()
        for sc in scales:
            a_blk.copy_(a_keep * sc)
            op.step(stream)
        op.drain()
        torch.cuda.synchronize()
        last = np.empty((m, n), np.float32)
        dev.memory_copy_from(op.buffers[(op.steps - 1) & 1], last, last.nbytes)
        prev = np.empty((m, n), np.float32)
        dev.memory_copy_from(op.buffers[(op.steps - 2) & 1], prev, prev.nbytes)
        assert np.array_equal(last, single * np.float32(scales[-1]))
        assert np.array_equal(prev, single * np.float32(scales[-2]))
        a_blk.copy_(a_keep)
        dist.barrier()
        loop = op.host_loop()
        host_c.fill_(float("nan"))
        a_blk.zero_()
        for _ in range(3):
            loop.submit(host_a.data_ptr(), host_c.data_ptr())
        loop.wait()
        dist.barrier()
        assert np.array_equal(host_c.numpy(), single[rank * rows:(rank + 1) * rows])
        assert np.array_equal(op.result(), single)
        loop.close()
        op.close()
        assert dev.status() == 0
        # ---- the same broadcast by NVLink multicast stores, where the box offers them ----
        # (no rank may fail while its memory is bound to the multicast object: compare, unbind
        # on every rank, and only then judge)
        op = PeerStoreMatmul(dev, a_blk.data_ptr(), b_dev.data_ptr(), m, n, k, world, rank,
                             config=pair_cfg, exchange="multimem?")
        used = op.exchange
        for _ in range(2):
            op.step(stream)
        torch.cuda.synchronize()
        dist.barrier()
        same = bool(np.array_equal(op.result(), single)) and dev.status() == 0
        op.close()
        verdict = torch.tensor([1.0 if same else 0.0], device="cuda")
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
        Path(out_dir, f"exchange{rank}").write_text(used)
        assert verdict.item() == 1.0, f"{used}: a rank's C differs from the single-GPU product"
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_row_sharded_matmul_on_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
    used = {(tmp_path / f"exchange{r}").read_text() for r in range(world)}
    assert len(used) == 1 and used <= {"multimem", "peer"}, used  # every rank took the same path
    print("fused all-gather ran by", used.pop())
