"""Row-sharded linear with kernel-side pushes, two ranks emulated on one GPU. Needs a B200.

Both "ranks" live in this process and their calls are issued one after the other on one stream,
so a kernel only ever waits for flags that an earlier, already finished launch has raised.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import tq1_oracle as o
from tests.gpu_util import random_blocks

pytestmark = pytest.mark.gpu


class TwoRanks:
    def __init__(self, rows, columns, batch):
        from ternel_b200 import _native
        from ternel_b200.sharding import ShardPlan
        self.lib = _native.lib()
        self.plan = ShardPlan(rows, 2)
        self.rows, self.columns, self.batch = rows, columns, batch
        self.y = [torch.zeros((batch, rows), dtype=torch.float16, device="cuda") for _ in range(2)]
        self.flags = [torch.zeros(rows // 16, dtype=torch.int32, device="cuda") for _ in range(2)]   # one per row tile
        self.base = torch.zeros(1, dtype=torch.int32, device="cuda")
        need = self.lib.tq1_linear_sharded_workspace_bytes(batch, rows // 2, columns)
        self.ws = [torch.zeros(need, dtype=torch.uint8, device="cuda") for _ in range(2)]

    def call(self, rank, blocks_dev, x_dev, publish, wait_epoch, wait=True):
        from ternel_b200 import _native
        from ternel_b200.sharding import make_shard
        shard = make_shard(rank=rank, plan=self.plan, peer_y=[t.data_ptr() for t in self.y],
                           peer_flags=[t.data_ptr() for t in self.flags], epoch_base=self.base.data_ptr(),
                           publish_epoch=publish, wait_epoch=wait_epoch,
                           wait_flags=self.flags[rank].data_ptr() if wait else None, wait_tiles=self.rows // 16)
        first, count = self.plan.rows(rank)
        rc = self.lib.tq1_linear_f16_sharded(
            blocks_dev[first:first + count].contiguous().data_ptr(), x_dev.data_ptr(), ctypes.byref(shard),
            self.batch, count, self.columns, self.ws[rank].data_ptr(), self.ws[rank].numel(),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, _native.last_error()


@pytest.mark.parametrize("batch", (1, 4))
@pytest.mark.parametrize(("rows", "columns"), ((1024, 5120), (5120, 1024)))
def test_shards_land_in_every_ranks_buffer(rows, columns, batch):
    blocks, rng = random_blocks(rows, columns, seed=rows + batch)
    blocks_dev = torch.from_numpy(blocks).cuda()
    ranks = TwoRanks(rows, columns, batch)
    for step in range(3):            # epochs keep growing: (1,2), (3,4), ...
        x = rng.standard_normal((batch, columns)).astype(np.float16)
        x_dev = torch.from_numpy(x).cuda()
        for rank in range(2):
            ranks.call(rank, blocks_dev, x_dev, publish=2 * step + 1, wait_epoch=2 * step)
        for rank in range(2):        # a dependent second call waits for the first call's flags of both ranks
            ranks.call(rank, blocks_dev, x_dev, publish=2 * step + 2, wait_epoch=2 * step + 1)
        torch.cuda.synchronize()
        want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
        for rank in range(2):
            got = ranks.y[rank].float().cpu().numpy()
            assert o.normalised_error(got, want) < 2e-3
            assert bool((ranks.flags[rank] == 2 * step + 2).all())          # every tile's flag, from both shards
            assert int(ranks.ws[rank][:8].view(torch.int32)[0]) == 0          # status word: no timeout
        assert torch.equal(ranks.y[0], ranks.y[1])


def test_a_flag_that_never_arrives_times_out_with_a_status():
    rows, columns = 256, 512
    blocks, rng = random_blocks(rows, columns, seed=1)
    ranks = TwoRanks(rows, columns, 1)
    x_dev = torch.from_numpy(rng.standard_normal((1, columns)).astype(np.float16)).cuda()
    ranks.call(0, torch.from_numpy(blocks).cuda(), x_dev, publish=1, wait_epoch=7)   # nobody publishes 7
    torch.cuda.synchronize()                                                          # returns: the wait is bounded
    assert int(ranks.ws[0][:4].view(torch.int32)[0]) == 4
    ranks.ws[0][:4].zero_()
    ranks.call(0, torch.from_numpy(blocks).cuda(), x_dev, publish=2, wait_epoch=0)   # the context is still usable
    torch.cuda.synchronize()
    assert int(ranks.ws[0][:4].view(torch.int32)[0]) == 0
