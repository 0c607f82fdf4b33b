"""Worker of tests/test_gpu_two_gpus.py: one process per GPU (torch.distributed.run, NCCL for set-up only).

(1) The batched sharded entry point (wait kernel, linear call, push kernel) across real NVLink: every rank's
    gathered buffer against the oracle, bit-equal between the ranks, every tile flag at its epoch.
(2) A two-layer decode chain with row- and column-sharded links: every link of every rank against the oracle.
"""

import ctypes
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from oracle import tq1_oracle as o                       # noqa: E402
from tests.gpu_util import random_blocks                 # noqa: E402


def sharded_calls(rank, world, device):
    import torch.distributed._symmetric_memory as symm_mem
    from ternel_b200 import _native
    from ternel_b200.sharding import ShardPlan, make_shard
    lib = _native.lib()
    for batch, rows, columns in ((1, 1024, 5120), (4, 1024, 5120), (4, 5120, 1024)):
        blocks, rng = random_blocks(rows, columns, seed=rows + batch)        # same bytes on every rank
        plan = ShardPlan(rows, world)
        first, count = plan.rows(rank)
        mine = torch.from_numpy(blocks[first:first + count].copy()).to(device)
        y = symm_mem.empty((batch, rows), dtype=torch.float16, device=device)
        flags = symm_mem.empty(rows // 16, dtype=torch.int32, device=device)
        y.zero_(); flags.zero_()
        hy, hf = symm_mem.rendezvous(y, dist.group.WORLD), symm_mem.rendezvous(flags, dist.group.WORLD)
        base = torch.zeros(1, dtype=torch.int32, device=device)
        need = lib.tq1_linear_sharded_workspace_bytes(batch, count, columns)
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        torch.cuda.synchronize(); dist.barrier()
        for step in range(3):
            x = rng.standard_normal((batch, columns)).astype(np.float16)
            x_dev = torch.from_numpy(x).to(device)
            for call in (1, 2):      # the second call waits for the first call's flags from both GPUs
                shard = make_shard(rank=rank, plan=plan, peer_y=[int(p) for p in hy.buffer_ptrs],
                                   peer_flags=[int(p) for p in hf.buffer_ptrs], epoch_base=base.data_ptr(),
                                   publish_epoch=2 * step + call, wait_epoch=2 * step + call - 1,
                                   wait_flags=flags.data_ptr(), wait_tiles=rows // 16)
                rc = lib.tq1_linear_f16_sharded(mine.data_ptr(), x_dev.data_ptr(), ctypes.byref(shard), batch, count,
                                                columns, ws.data_ptr(), ws.numel(),
                                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                assert rc == 0, _native.last_error()
            torch.cuda.synchronize(); dist.barrier()
            want = o.float64_matmul(blocks, x, rows=rows, columns=columns)
            got = y.float().cpu().numpy()
            assert o.normalised_error(got, want) < 2e-3, (rank, batch, rows, columns)
            assert bool((flags == 2 * step + 2).all()), "a tile flag did not reach its epoch"
            assert int(ws[:4].view(torch.int32)[0]) == 0, "a bounded wait ran out"
            both = [torch.empty_like(y) for _ in range(world)]
            dist.all_gather(both, y.contiguous())
            assert all(torch.equal(both[0], b) for b in both), "the ranks' gathered buffers differ"
            dist.barrier()
    return "sharded calls ok"


def chain(rank, world, device):
    from bench import verify_chain
    from ternel_b200.stack import LayerStack
    stack = LayerStack(layers=2, batch=1, vocab=4096, rank=rank, world=world, device=device, seed=3, fused=True)
    assert stack.column_sharded("o", 0) and stack.column_sharded("down", 0) and not stack.column_sharded("down", 1)
    for _ in range(2):
        dist.barrier(); stack.step(); torch.cuda.synchronize()
    assert stack.status() == 0
    parity = verify_chain(stack, world, rank)
    assert parity["ranks_checked"] == world and parity["max_err"] < 2e-3
    return f"chain ok {parity['max_err']:.2e}"


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    try:
        messages = [sharded_calls(rank, world, device), chain(rank, world, device)]
        dist.barrier()
        if rank == 0:
            print("TWO_GPU_WORKER_OK", *messages, flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
