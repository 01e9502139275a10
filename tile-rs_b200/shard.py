"""How each operator splits across GPUs: independent units, no exchange step.

The unit is the per-block tile of ``#[tile_kernel]``
(crates/tile_std_macros/src/lib.rs:237-254): softmax rows, GEMM batches,
attention (batch, KV-head) groups.  A single large GEMM is split by N-column
blocks instead, each rank receiving its columns of B as a contiguous [K, N/G]
matrix.  The reference itself is single-device
(crates/tile_hal/src/backend.rs:95-112).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import capi


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


def softmax_rows(rows: int, world: int, rank: int) -> Shard:
    return shard_range(rows, world, rank)


def gemm_batches(batch: int, world: int, rank: int) -> Shard:
    return shard_range(batch, world, rank)


def gemm_n_columns(n: int, world: int, rank: int, granule: int = 256) -> Shard:
    """Column range [first, stop) of C (and B) for ``rank``; multiples of ``granule`` (one N tile)."""
    blocks = (n + granule - 1) // granule
    s = shard_range(blocks, world, rank)
    first = min(s.first * granule, n)
    stop = min(s.stop * granule, n)
    return Shard(first, stop - first)


def attention_groups(batch: int, heads_kv: int, world: int, rank: int) -> Shard:
    """(batch, KV-head) groups, flattened batch-major, owned by ``rank``."""
    return shard_range(batch * heads_kv, world, rank)
