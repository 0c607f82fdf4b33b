"""Host logic of the row sharding, and a two-rank gloo run of shard -> gather on CPU (no GPU)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import c_oracle, tq1_oracle as o
from ternel_b200.sharding import EpochClock, ShardPlan, make_shard


def test_shard_plan_partitions_rows_and_bytes():
    for n, world in ((5120, 8), (34816, 8), (7168, 4), (1024, 2), (17408, 1)):
        plan = ShardPlan(n, world)
        covered = []
        for r in range(world):
            first, count = plan.rows(r)
            assert first % 16 == 0 and count == n // world
            covered.extend(range(first, first + count))
            lo, hi = plan.byte_range(r, 5120)
            assert lo == first * 1120 and hi - lo == count * 1120
        assert covered == list(range(n))
    with pytest.raises(ValueError, match="do not shard evenly"):
        ShardPlan(1000, 3)
    with pytest.raises(ValueError, match="multiple of 16"):
        ShardPlan(1000, 5)
    with pytest.raises(ValueError, match="between 1 and 8"):
        ShardPlan(1024, 16)
    with pytest.raises(ValueError, match="outside"):
        ShardPlan(1024, 2).rows(2)


def test_epoch_clock_and_shard_struct():
    clock = EpochClock()
    assert [clock.next() for _ in range(3)] == [(1, 0), (2, 1), (3, 2)]
    assert clock.reset() == 3 and clock.next() == (1, 0)
    plan = ShardPlan(1024, 2)
    shard = make_shard(rank=1, plan=plan, peer_y=[0x1000, 0x2000], peer_flags=[0x100, 0x200], epoch_base=0x300,
                       publish_epoch=5, wait_epoch=4, wait_flags=0x200, wait_tiles=64)
    assert (shard.rank, shard.world, shard.n_offset, shard.n_total) == (1, 2, 512, 1024)
    assert shard.peer_y[1] == 0x2000 and shard.wait_flags == 0x200 and shard.epoch_base == 0x300
    assert shard.wait_tiles == 64
    nowait = make_shard(rank=0, plan=plan, peer_y=[1, 2], peer_flags=[3, 4], epoch_base=0, publish_epoch=1,
                        wait_epoch=0)
    assert not nowait.wait_flags and nowait.wait_tiles == 0
    with pytest.raises(ValueError, match="per rank"):
        make_shard(rank=0, plan=plan, peer_y=[1], peer_flags=[1, 2], epoch_base=0, publish_epoch=1, wait_epoch=0)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, result_queue) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, columns, batch = 512, 1024, 3
        blocks, x = None, None
        rng = np.random.default_rng(5)             # same seed everywhere: every rank builds the whole weight
        groups = rows * columns // 128
        trits = rng.integers(0, 3, size=(groups, 128), dtype=np.uint8)
        scales = rng.normal(0.0, 0.05, size=groups).astype(np.float16)
        blocks = o.encode_blocks(scales.view(np.uint8).reshape(-1, 2), trits).reshape(rows, columns // 128, 28)
        x = rng.standard_normal((batch, columns)).astype(np.float16).astype(np.float32)
        plan = ShardPlan(rows, world)
        first, count = plan.rows(rank)
        lo, hi = plan.byte_range(rank, columns)
        mine = blocks.reshape(-1)[lo:hi].reshape(count, columns // 128, 28)       # the shard is a byte range
        assert np.array_equal(mine, blocks[first:first + count])
        y_local = torch.from_numpy(c_oracle.matmul_f32(mine, x, rows=count, columns=columns, threads=1))
        pieces = [torch.empty((batch, count), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(pieces, y_local.contiguous())
        full = torch.cat(pieces, dim=1).numpy()
        want = c_oracle.matmul_f32(blocks, x, rows=rows, columns=columns, threads=1)
        result_queue.put((rank, bool(np.array_equal(full, want))))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_then_gather_equals_the_whole():
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {0: True, 1: True}


def test_column_shards_only_where_a_rank_gets_whole_chunks():
    """Which projections of the decode stack are sharded by columns (pure shape logic, no GPU): o and down, except
    the last down, and only where K / world is a whole number of 512-column chunks; the shard shapes follow."""
    from ternel_b200.stack import LayerShape, LayerStack

    class Shapes(LayerStack):
        def __init__(self, world, layers=3):
            self.world, self.layers, self.column_shards = world, layers, world > 1
            self.projections = LayerShape().projections(True)

    one, two, four = Shapes(1), Shapes(2), Shapes(4)
    assert not any(one.column_sharded(name, 0) for name, _, _ in one.projections)
    assert [two.column_sharded(name, 0) for name, _, _ in two.projections] == [False, True, False, True]
    assert not two.column_sharded("down", 2)                      # the step's result stays a row shard
    assert two.shard_shape("o", 5120, 5120, 0) == (5120, 2560)
    assert two.shard_shape("down", 5120, 17408, 0) == (5120, 8704)
    assert two.shard_shape("down", 5120, 17408, 2) == (2560, 17408)
    assert two.shard_shape("qkv", 7168, 5120, 0) == (3584, 5120)
    # 5120 / 4 = 1280 and 17408 / 4 = 4352 are not multiples of 512: rows
    assert not any(four.column_sharded(name, 0) for name, _, _ in four.projections)
    assert four.shard_shape("o", 5120, 5120, 0) == (1280, 5120)
