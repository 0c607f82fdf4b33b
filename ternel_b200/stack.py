"""A stack of packed decoder-layer projections resident on one GPU.

This is the decode-step harness used by the benchmark and the multi-GPU tests:
``layers`` copies of the seven projections of a dense decoder layer (q, k, v,
o, gate, up, down), each a ``PackedLinear``-shaped weight of canonical blocks,
optionally output-row-sharded over the ranks of a process group. One ``step``
streams every weight byte once (the batch-1 / small-batch regime of
src/ternel_mlx/modules.py:425-457 of the reference, where a decoded token issues
one matmul per linear leaf), gathers one embedding row per sequence, and, when
sharded, all-gathers each projection's output shards so every rank holds the
whole activation again.

Inputs of the projections are fixed synthetic activations (no attention or
normalisation sits between them here), so the values stay finite while the
launch order and the bytes moved are those of a real decode step.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native
from .format import BLOCK_BYTES, BLOCK_SIZE, check


@dataclass(frozen=True)
class LayerShape:
    hidden: int = 5120
    ffn: int = 17408
    q_heads: int = 40
    kv_heads: int = 8
    head_dim: int = 128

    def projections(self, fused: bool = False) -> tuple[tuple[str, int, int], ...]:
        """(name, N out, K in) in launch order.

        ``fused`` stores q/k/v (same input) as one row-concatenated matrix and gate/up
        likewise, as fused-QKV checkpoints do: the same bytes in four launches per layer
        instead of seven.
        """
        q = self.q_heads * self.head_dim
        kv = self.kv_heads * self.head_dim
        if fused:
            return (("qkv", q + 2 * kv, self.hidden), ("o", self.hidden, q),
                    ("gate_up", 2 * self.ffn, self.hidden), ("down", self.hidden, self.ffn))
        return (
            ("q", q, self.hidden), ("k", kv, self.hidden), ("v", kv, self.hidden),
            ("o", self.hidden, q), ("gate", self.ffn, self.hidden), ("up", self.ffn, self.hidden),
            ("down", self.hidden, self.ffn),
        )

    def packed_bytes_per_layer(self) -> int:
        return sum(n * k // BLOCK_SIZE * BLOCK_BYTES for _, n, k in self.projections())


def random_blocks_device(rows: int, columns: int, generator: torch.Generator, device,
                         p_zero: float = 0.40) -> torch.Tensor:
    """Random legal canonical blocks built on the GPU with the benchmark's distributions:
    trits -1/0/+1 with P = (1-p0)/2, p0, (1-p0)/2 and one FP16 scale |N(0,1)|*0.02 per group."""
    groups = rows * columns // BLOCK_SIZE
    out = torch.empty((groups, BLOCK_BYTES), dtype=torch.uint8, device=device)
    lo, hi = (1 - p_zero) / 2, (1 + p_zero) / 2
    pow5 = torch.tensor([1, 3, 9, 27, 81], dtype=torch.int16, device=device)
    chunk = 1 << 18
    for g0 in range(0, groups, chunk):
        n = min(chunk, groups - g0)
        u = torch.rand((n, BLOCK_SIZE), generator=generator, device=device)
        trits = (u >= lo).to(torch.int16) + (u >= hi).to(torch.int16)
        full = (trits[:, :125].reshape(n, 25, 5) * pow5).sum(dim=2)
        tail = (trits[:, 125:] * pow5[:3]).sum(dim=1)
        scale = (torch.randn(n, generator=generator, device=device).abs() * 0.02).to(torch.float16)
        out[g0:g0 + n, 0:2] = scale.view(torch.uint8).reshape(n, 2)
        out[g0:g0 + n, 2:27] = full.to(torch.uint8)
        out[g0:g0 + n, 27] = tail.to(torch.uint8)
    return out.reshape(rows, columns // BLOCK_SIZE, BLOCK_BYTES)


class LayerStack:
    """``layers`` x 7 packed projections (+ an embedding table), row-sharded over ``world`` ranks."""

    def __init__(self, *, layers: int, batch: int = 1, shape: LayerShape = LayerShape(),
                 vocab: int = 0, rank: int = 0, world: int = 1, device=None, seed: int = 0,
                 group=None, fused: bool = False, exchange: str = "p2p", weights_from: "LayerStack | None" = None) -> None:
        self.layers, self.batch, self.shape = layers, batch, shape
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device if device is not None else "cuda")
        self.lib = _native.lib()
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed * 1000 + rank)
        self.fused = fused
        self.projections = shape.projections(fused)
        for _, n, _ in self.projections:
            if n % world or (n // world) % 16:
                raise ValueError(f"{n} output rows do not shard evenly over {world} ranks")
        # weights[l][j]: this rank's rows [rank*N/P, (rank+1)*N/P) of projection j in layer l
        if weights_from is not None:       # a second stack (another batch size) over the same resident weights
            if (weights_from.projections, weights_from.world, weights_from.layers) != (self.projections, world, layers):
                raise ValueError("weights_from must have the same layers, projections and sharding")
            self.weights = weights_from.weights
        else:
            self.weights = [[random_blocks_device(n // world, k, gen, self.device) for _, n, k in self.projections]
                            for _ in range(layers)]
        xg = torch.Generator(device=self.device)
        xg.manual_seed(seed + 7)   # same activations on every rank
        self.inputs = {k: torch.randn((batch, k), generator=xg, device=self.device).to(torch.float16)
                       for k in sorted({k for _, _, k in self.projections})}
        # full-width outputs; a rank computes its slice [.., rank*N/P:(rank+1)*N/P] and gathers the rest
        self.shards = {n: torch.zeros((batch, n // world), dtype=torch.float16, device=self.device)
                       for n in sorted({n for _, n, _ in self.projections})}
        self.outputs = {n: torch.zeros((world, batch, n // world), dtype=torch.float16, device=self.device)
                        for n in sorted({n for _, n, _ in self.projections})}
        self.vocab = vocab
        if vocab:
            self.table = (weights_from.table if weights_from is not None and weights_from.vocab == vocab
                          else random_blocks_device(vocab, shape.hidden, gen, self.device))
            self.ids = torch.randint(0, vocab, (batch,), generator=xg, device=self.device)
            self.embedded = torch.zeros((batch, shape.hidden), dtype=torch.float16, device=self.device)
        ws_bytes = max(self.lib.tq1_linear_workspace_bytes(batch, n // world, k) for _, n, k in self.projections)
        self.workspace = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=self.device)
        self.workspace_bytes = ws_bytes
        self.launches_per_step = layers * len(self.projections) + (1 if vocab else 0)
        self.exchange = exchange if world > 1 else "none"
        if self.exchange == "p2p":
            self._setup_peer_buffers()

    def _setup_peer_buffers(self) -> None:
        """Gathered outputs and flags in symmetric memory so every rank can write into every other's."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        from .sharding import EpochClock, ShardPlan

        sizes = sorted({n for _, n, _ in self.projections})
        # arena: [epoch base 4 B | pad to 1 KiB] then, per output size, the gathered buffer and its tile flags
        self._offsets, self._flag_offsets, cursor = {}, {}, 1024
        for n in sizes:
            self._offsets[n] = cursor
            cursor += (self.batch * n * 2 + 255) // 256 * 256
            self._flag_offsets[n] = cursor
            cursor += (n // 16 * 4 + 255) // 256 * 256
        arena = symm_mem.empty(cursor, dtype=torch.uint8, device=self.device)
        arena.zero_()
        handle = symm_mem.rendezvous(arena, self.group if self.group is not None else dist.group.WORLD)
        self._arena, self._handle = arena, handle
        self._peer_base = [int(p) for p in handle.buffer_ptrs]
        self.outputs = {n: arena[self._offsets[n]: self._offsets[n] + self.batch * n * 2].view(torch.float16)
                        .view(self.batch, n) for n in sizes}
        self._plans = {n: ShardPlan(n, self.world) for n in sizes}
        self._clock = EpochClock()
        self._epoch_base_ptr = self._peer_base[self.rank]
        ws_bytes = max(self.lib.tq1_linear_sharded_workspace_bytes(self.batch, n // self.world, k)
                       for _, n, k in self.projections)
        self.workspace = torch.zeros(ws_bytes, dtype=torch.uint8, device=self.device)
        self.workspace_bytes = ws_bytes
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------
    @property
    def packed_bytes_per_step(self) -> int:
        """Packed weight bytes this rank streams per step."""
        return self.layers * self.shape.packed_bytes_per_layer() // self.world

    @property
    def algorithmic_bytes_per_step(self) -> int:
        """Packed weights + FP16 activations in + FP16 outputs out, this rank, one step."""
        total = 0
        for _, n, k in self.projections:
            total += (n // self.world) * k // BLOCK_SIZE * BLOCK_BYTES + 2 * self.batch * (k + n // self.world)
        total *= self.layers
        if self.vocab:
            total += self.batch * (self.shape.hidden // BLOCK_SIZE * BLOCK_BYTES + 2 * self.shape.hidden)
        return total

    def step(self) -> None:
        """Enqueue one decode step on the current stream (no synchronisation)."""
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        lib, batch, world = self.lib, self.batch, self.world
        ws, ws_bytes = self.workspace.data_ptr(), self.workspace_bytes
        if self.vocab:
            check(lib.tq1_embedding_f16(self.table.data_ptr(), self.ids.data_ptr(), self.embedded.data_ptr(),
                                        0, batch, self.vocab, self.shape.hidden, stream))
        if self.exchange == "p2p":
            self._step_p2p(stream)
            return
        for layer in self.weights:
            for (_, n, k), blocks in zip(self.projections, layer):
                if world == 1:
                    y = self.outputs[n]
                    check(lib.tq1_linear_f16(blocks.data_ptr(), self.inputs[k].data_ptr(), y.data_ptr(), 0,
                                             batch, n, k, ws, ws_bytes, stream))
                else:
                    shard = self.shards[n]
                    check(lib.tq1_linear_f16(blocks.data_ptr(), self.inputs[k].data_ptr(), shard.data_ptr(), 0,
                                             batch, n // world, k, ws, ws_bytes, stream))
                    torch.distributed.all_gather_into_tensor(self.outputs[n], shard, group=self.group)

    def _step_p2p(self, stream) -> None:
        """Every projection pushes its rows into all ranks' gathered buffers; the next one waits for the flags."""
        from .sharding import make_shard, sharded_linear
        lib, world, rank = self.lib, self.world, self.rank
        local = self._peer_base[rank]
        prev_n = self.projections[-1][1]          # a step starts after the previous step's last projection
        for layer in self.weights:
            for (_, n, k), blocks in zip(self.projections, layer):
                publish, wait = self._clock.next()
                # the input stands for the previous projection's gathered output: wait for the tiles of
                # that buffer which cover this projection's K columns
                shard = make_shard(rank=rank, plan=self._plans[n],
                                   peer_y=[base + self._offsets[n] for base in self._peer_base],
                                   peer_flags=[base + self._flag_offsets[n] for base in self._peer_base],
                                   epoch_base=self._epoch_base_ptr, publish_epoch=publish, wait_epoch=wait,
                                   wait_flags=local + self._flag_offsets[prev_n], wait_tiles=min(k, prev_n) // 16)
                sharded_linear(lib, blocks.data_ptr(), self.inputs[k].data_ptr(), shard, batch=self.batch,
                               n_local=n // world, columns=k, workspace_ptr=self.workspace.data_ptr(),
                               workspace_bytes=self.workspace_bytes, stream_ptr=stream)
                prev_n = n
        check(lib.tq1_shard_advance_epoch(self._epoch_base_ptr, self._clock.reset(), stream))

    def checksum(self) -> float:
        """Consumes every output so the work cannot be dead-coded; also a cross-rank equality check."""
        return float(sum(v.float().abs().sum() for v in self.outputs.values()))
