"""The process-per-GPU form of the multi-GPU path on CPU ranks (gloo): every rank derives its
shard from (world, rank) alone, shards tile the whole problem, the verification gather
reassembles the full result in unit order, a rank whose shard is wrong is found and named, and
a rank that leaves before its launch is noticed on the host instead of being waited for."""
import datetime
import os
import socket
import sys
import zlib
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _setup(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import __graft_entry__ as entry
    import util
    return entry.load_package(), entry.load_oracle(), util


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, corrupt_rank):
    pkg, oracle, util = _setup(rank, world, port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols = 37, 64  # ragged on purpose
        sh = pkg.launcher.shard_range(rows, world, rank)
        # each rank generates only its rows of the seeded stream ...
        x = util.gen_normal(pkg.capi, (sh.count, cols), 201, 3.0, first=sh.first * cols)
        y = oracle.softmax_f32(x) if sh.count else np.zeros((0, cols), np.float32)  # CPU stand-in for the kernel
        if rank == corrupt_rank:
            y[0, 0] += 1e-3  # a shard that came back wrong
        # ... and the verification gather (NCCL on GPUs, gloo here) reassembles them in order
        parts = [None] * world
        dist.all_gather_object(parts, (rank, sh.first, y, zlib.crc32(y.tobytes())))
        full = np.concatenate([p[2] for p in sorted(parts, key=lambda t: t[1])])
        ref = oracle.softmax_f32(util.gen_normal(pkg.capi, (rows, cols), 201, 3.0))
        assert full.shape == ref.shape
        # every rank checks every shard's checksum against the reference's rows for that shard
        bad = [r for r, first, part, crc in parts if crc != zlib.crc32(ref[first:first + len(part)].tobytes())]
        assert bad == ([corrupt_rank] if corrupt_rank >= 0 else []), bad
        if corrupt_rank < 0:
            assert np.array_equal(full, ref)
        # max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        # GEMM N-column split: the column blocks tile [0, N) in whole 256-column tiles
        job = pkg.launcher.gemm_job(pkg.capi.BF16, 8192, 8192, 8192, 0, 0, 0)
        cols_sh = [job.plan(world, r) for r in range(world)]
        assert cols_sh[0].first == 0 and cols_sh[-1].stop == 8192 and all(c.first % 256 == 0 for c in cols_sh)
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_gather(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), -1), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_a_wrong_shard_is_found_and_named(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), 1), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def _leaver(rank, world, port, out_dir):
    """Rank 1 leaves between steps, before its launch.  Rank 0 learns of it on the host (a heartbeat key in
    the store that never appears) within a short limit and says which rank is missing."""
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=20))
    store.set(f"joined{rank}", "1")
    store.wait([f"joined{r}" for r in range(world)])
    if rank == 1:
        store.set("left1", "1")  # orderly: nothing of this rank is in flight
        return
    store.set(f"step1_ready{rank}", "1")
    missing = []
    for r in range(world):
        try:
            store.wait([f"step1_ready{r}"], datetime.timedelta(milliseconds=500))
        except Exception:
            missing.append(r)
    assert missing == [1], missing
    assert store.get("left1") == b"1"
    (Path(out_dir) / "noticed").write_text(f"rank {missing[0]} did not reach step 1")


def test_a_rank_that_leaves_before_launch_is_noticed(tmp_path):
    mp.spawn(_leaver, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "noticed").read_text() == "rank 1 did not reach step 1"
