"""Output-row sharding of packed projections over the GPUs of one node.

Output rows of a packed linear are independent (each ``y[n]`` touches only row ``n``'s
blocks), so rank ``r`` owns rows ``[r*N/P, (r+1)*N/P)`` of every projection: a contiguous byte
range of the canonical weight. After a sharded projection every rank needs the whole FP16
result again. This module serves the batched kernels (two or more activation rows):

* ``tq1_linear_f16_sharded``: a wait kernel (bounded spin on the tile flags of the activations
  the call reads), the ordinary linear call on this rank's rows, and a push kernel that writes
  the rows straight into every rank's gathered buffer over NVLink peer mappings and then raises
  a per-tile flag there. No collective kernel runs.
* the baseline is ``all_gather_into_tensor`` after each projection.

Batch-1 decode shards inside the chain kernel instead (``ternel_b200.chain.ChainPlan`` with
``peers``): outputs travel between projections and between GPUs as tagged 64-bit words.

The reference is single-device (patches/prism-tq1-g128-distribution.patch:373), so this module
has no counterpart there; the layout it shards is the reference's canonical block array.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

from . import _native

ROW_QUANTUM = 16          # shard boundaries fall on row-tile boundaries of the kernels
MAX_RANKS = 8


@dataclass(frozen=True)
class ShardPlan:
    """Row ranges of one projection's output over ``world`` ranks (pure host logic)."""

    n_total: int
    world: int

    def __post_init__(self) -> None:
        if not 1 <= self.world <= MAX_RANKS:
            raise ValueError(f"world size must be between 1 and {MAX_RANKS}, got {self.world}")
        if self.n_total <= 0 or self.n_total % self.world:
            raise ValueError(f"{self.n_total} output rows do not shard evenly over {self.world} ranks")
        if (self.n_total // self.world) % ROW_QUANTUM:
            raise ValueError(
                f"{self.n_total // self.world} rows per rank is not a multiple of {ROW_QUANTUM}")

    @property
    def rows_per_rank(self) -> int:
        return self.n_total // self.world

    def rows(self, rank: int) -> tuple[int, int]:
        """(first row, row count) owned by ``rank``."""
        if not 0 <= rank < self.world:
            raise ValueError(f"rank {rank} outside [0, {self.world})")
        return rank * self.rows_per_rank, self.rows_per_rank

    def byte_range(self, rank: int, columns: int) -> tuple[int, int]:
        """Byte range of the rank's rows inside the canonical block array of a ``K = columns`` weight."""
        first, count = self.rows(rank)
        row_bytes = columns // 128 * 28
        return first * row_bytes, (first + count) * row_bytes


class EpochClock:
    """Publish/wait epochs of consecutive sharded calls (identical on every rank).

    Call ``i`` (1-based within a step) publishes epoch ``i`` and waits for epoch ``i-1`` of the
    call before it; a device-side base that advances by ``calls_per_step`` each step keeps the
    values fresh when a captured step is replayed.
    """

    def __init__(self) -> None:
        self.calls = 0

    def next(self) -> tuple[int, int]:
        """(publish_epoch, wait_epoch) for the next call of the step."""
        self.calls += 1
        return self.calls, self.calls - 1

    def reset(self) -> int:
        """End of a step: returns how far the device-side base must advance."""
        calls, self.calls = self.calls, 0
        return calls


def make_shard(*, rank: int, plan: ShardPlan, peer_y: list[int], peer_flags: list[int], epoch_base: int,
               publish_epoch: int, wait_epoch: int, wait_flags: int | None = None,
               wait_tiles: int | None = None) -> _native.Shard:
    """Fill a ``tq1_shard`` for one call.

    ``peer_y[p]`` / ``peer_flags[p]`` are device addresses on rank p of the gathered output and of its
    tile flags (one 32-bit word per 16 rows). ``wait_flags`` is the local flag array of the buffer the
    activations were gathered into (``wait_tiles`` words); ``None`` skips the wait.
    """
    if len(peer_y) != plan.world or len(peer_flags) != plan.world:
        raise ValueError("one gathered buffer and one flag array per rank are required")
    first, _ = plan.rows(rank)
    shard = _native.Shard()
    shard.rank, shard.world = rank, plan.world
    shard.n_offset, shard.n_total = first, plan.n_total
    for p in range(plan.world):
        shard.peer_y[p] = peer_y[p]
        shard.peer_flags[p] = peer_flags[p]
    shard.epoch_base = epoch_base or None
    shard.publish_epoch = publish_epoch
    shard.wait_flags = wait_flags or None
    shard.wait_tiles = int(wait_tiles or 0) if wait_flags else 0
    shard.wait_epoch = wait_epoch
    return shard


def sharded_linear(lib, blocks_ptr: int, x_ptr: int, shard: _native.Shard, *, batch: int, n_local: int,
                   columns: int, workspace_ptr: int, workspace_bytes: int, stream_ptr: int) -> None:
    from .format import check
    check(lib.tq1_linear_f16_sharded(blocks_ptr, x_ptr, ctypes.byref(shard), batch, n_local, columns,
                                     workspace_ptr, workspace_bytes, stream_ptr))
