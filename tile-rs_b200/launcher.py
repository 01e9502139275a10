"""Multi-GPU launcher: one problem, described once on host buffers, run on a list of devices.

Host-side mirror of ``tsm100_multi_run``.  The reference's HAL drives one GPU per process
(crates/tile_hal/src/cuda.rs:321-327, crates/tile_hal/src/backend.rs:95-112); the hot path
has no exchange step, so a problem is dealt out in independent units - the per-block tiles of
``#[tile_kernel]`` (crates/tile_std_macros/src/lib.rs:237-254): softmax rows, GEMM problems of
a batch or N-column blocks of one large GEMM, attention (batch, KV-head) groups.  Every device
gets a host thread, a stream and a workspace of its own; no device reads another's memory and
there is no collective.

``shard_range`` is the same split for the process-per-GPU form (one rank per device under
``torch.distributed``): a rank derives its shard from (world, rank) alone.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

from . import capi, hal


@dataclass(frozen=True)
class Shard:
    first: int
    count: int

    @property
    def stop(self) -> int:
        return self.first + self.count


def shard_range(units: int, world: int, rank: int) -> Shard:
    """Contiguous block of ``units`` owned by ``rank``; the first ``units % world`` ranks get one more."""
    first, count = C.c_int64(), C.c_int64()
    st = capi.lib().tsm100_shard_range(units, world, rank, C.byref(first), C.byref(count))
    if st != capi.OK:
        raise ValueError(capi.last_error())
    return Shard(first.value, count.value)


@dataclass
class Report:
    """What one device did (``tsm100_multi_report``)."""
    ordinal: int
    status: int
    first: int
    count: int
    upload_ms: float
    kernel_ms: float
    download_ms: float
    total_ms: float
    device_status: int
    message: str


class Job:
    """A ``tsm100_multi_job`` that keeps its descriptor alive."""

    def __init__(self, op: int, desc, inputs: Sequence[int], out: int, launches: int = 1, timeout_ms: int = 0):
        self.desc = desc
        ins = (capi.c_vp * 3)(*[(p or None) for p in list(inputs) + [0] * (3 - len(inputs))])
        self.raw = capi.MultiJob(op, C.cast(C.pointer(desc), capi.c_vp), ins, out or None, launches, timeout_ms)

    def plan(self, n: int, index: int) -> Shard:
        """The shard device ``index`` of ``n`` gets (``tsm100_multi_plan``)."""
        first, count = C.c_int64(), C.c_int64()
        hal.check(capi.lib().tsm100_multi_plan(C.byref(self.raw), n, index, C.byref(first), C.byref(count)))
        return Shard(first.value, count.value)


def softmax_job(dtype, rows, cols, x, y, **kw) -> Job:
    return Job(capi.OP_SOFTMAX, capi.SoftmaxDesc(dtype, rows, cols), [x], y, **kw)


def gemm_job(dtype, m, n, k, a, b, c, *, out_dtype=None, b_transposed=False, batch=1, lda=0, ldb=0, ldc=0, **kw) -> Job:
    d = capi.GemmDesc(dtype, dtype if out_dtype is None else out_dtype, int(b_transposed), batch, m, n, k, lda, ldb, ldc)
    return Job(capi.OP_GEMM, d, [a, b], c, **kw)


def attention_job(dtype, batch, heads_q, heads_kv, seq, head_dim, q, k, v, o, *, causal=False, **kw) -> Job:
    d = capi.AttentionDesc(dtype, int(causal), batch, heads_q, heads_kv, seq, head_dim)
    return Job(capi.OP_ATTENTION, d, [q, k, v], o, **kw)


class MultiGpuLauncher:
    """Runs jobs on a fixed list of device ordinals.  ``run`` raises ``HalError`` naming the first
    device that failed; the per-device reports of the last run stay in ``last_reports`` either way."""

    def __init__(self, ordinals: Sequence[int]):
        if not ordinals:
            raise ValueError("empty device list")
        self.ordinals = list(ordinals)
        self.last_reports: List[Report] = []

    def run(self, job: Job, worker: Optional[Callable] = None) -> List[Report]:
        """``worker(job, ordinal, first, count, report) -> status`` replaces the built-in CUDA worker
        (``tsm100_multi_run_with``); the split, the threads, the clock watching and the reports are
        the launcher's either way."""
        n = len(self.ordinals)
        ords = (capi.c_i32 * n)(*self.ordinals)
        reps = (capi.MultiReport * n)()
        lib = capi.lib()
        if worker is None:
            st = lib.tsm100_multi_run(C.byref(job.raw), ords, n, reps)
        else:
            def tramp(_user, jobp, ordinal, first, count, rep):
                try:
                    return int(worker(jobp.contents, ordinal, first, count, rep.contents))
                except Exception as exc:  # a worker that raises is a failed device, not a crashed launcher
                    rep.contents.message = str(exc).encode()[:159]
                    return capi.ERR_RUNTIME
            cb = capi.MULTI_WORKER_FN(tramp)
            st = lib.tsm100_multi_run_with(C.byref(job.raw), ords, n, reps, cb, None)
        self.last_reports = [Report(r.ordinal, r.status, r.first, r.count, r.upload_ms, r.kernel_ms, r.download_ms,
                                    r.total_ms, r.device_status, r.message.decode(errors="replace")) for r in reps]
        hal.check(st)
        return self.last_reports

    @staticmethod
    def release() -> None:
        """Frees the per-device workspaces the launcher keeps between runs."""
        hal.check(capi.lib().tsm100_multi_release())
