"""The multi-GPU launch logic on two CPU ranks (gloo): every rank derives its shard
from (world, rank) alone, shards tile the whole problem, and the verification
gather reassembles the full result in unit order."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import __graft_entry__ as entry
    import util
    pkg = entry.load_package()
    oracle = entry.load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols = 37, 64  # ragged on purpose
        sh = pkg.shard.softmax_rows(rows, world, rank)
        # each rank generates only its rows of the seeded stream ...
        x = util.gen_normal(pkg.capi, (sh.count, cols), 201, 3.0, first=sh.first * cols)
        y = oracle.softmax_f32(x) if sh.count else np.zeros((0, cols), np.float32)  # CPU stand-in for the kernel
        # ... and the verification gather (NCCL on GPUs, gloo here) reassembles them in order
        parts = [None] * world
        dist.all_gather_object(parts, (sh.first, y))
        full = np.concatenate([p[1] for p in sorted(parts, key=lambda t: t[0])])
        ref = oracle.softmax_f32(util.gen_normal(pkg.capi, (rows, cols), 201, 3.0))
        assert full.shape == ref.shape and np.array_equal(full, ref)
        # max-over-ranks timing reduction used by the benchmark
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        # GEMM N-column split: the column blocks tile [0, N)
        cols_sh = [pkg.shard.gemm_n_columns(8192, world, r) for r in range(world)]
        assert cols_sh[0].first == 0 and cols_sh[-1].stop == 8192
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_and_gather(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
