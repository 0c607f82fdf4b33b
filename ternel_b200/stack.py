"""A stack of packed decoder-layer projections resident on one GPU.

This is the decode-step harness used by the benchmark and the multi-GPU tests:
``layers`` copies of the projections of a dense decoder layer (q, k, v, o, gate,
up, down), each a ``PackedLinear``-shaped weight of canonical blocks, optionally
output-row-sharded over the ranks of a process group. One ``step`` streams every
weight byte once (the batch-1 / small-batch regime of
src/ternel_mlx/modules.py:425-457 of the reference, where a decoded token issues
one matmul per linear leaf) and gathers one embedding row per sequence.

Exchange modes:

* ``"chain"`` (batch 1): the whole step is ONE persistent launch
  (``ternel_b200.chain.ChainPlan``). Projections depend on each other the way a
  decoder's do: q|k|v reads the previous layer's output (the embedding row for the
  first layer), o reads the q part of q|k|v, gate|up reads o and applies
  ``silu(gate) * up`` in its epilogue, down reads that. No attention or
  normalisation sits in between, so every link carries an output scale that keeps
  the activations at unit scale through all layers. With several ranks every
  finished output is pushed into every rank's hand-off area by the kernel itself
  (symmetric memory, plain peer stores).
* ``"launches"``: one launch per projection over fixed synthetic inputs (any
  batch); with several ranks the shards are all-gathered by NCCL after each
  projection (the baseline exchange).
"""

from __future__ import annotations

import ctypes
import math
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


def unit_gain(columns: int, p_zero: float = 0.40, scale_second_moment: float = 0.02 ** 2) -> float:
    """Output scale that keeps a unit-RMS activation vector at unit RMS through a random packed linear:
    the output variance is ``columns * P(nonzero) * E[scale^2]`` times the input's."""
    return 1.0 / math.sqrt(columns * (1.0 - p_zero) * scale_second_moment)


def swiglu_gain(pre_rms: float) -> float:
    """1 / RMS of ``silu(g) * u`` for independent ``g, u ~ N(0, pre_rms^2)`` (fixed-seed Monte Carlo, so
    that every rank computes the same number)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1234)
    g = torch.randn(1 << 20, generator=gen, dtype=torch.float64) * pre_rms
    u = torch.randn(1 << 20, generator=gen, dtype=torch.float64) * pre_rms
    return 1.0 / float(((g / (1 + torch.exp(-g)) * u) ** 2).mean().sqrt())


class LayerStack:
    """``layers`` x the projections of a decoder layer (+ an embedding table), row-sharded over ``world`` ranks."""

    def __init__(self, *, layers: int, batch: int = 1, shape: LayerShape = LayerShape(),
                 vocab: int = 0, rank: int = 0, world: int = 1, device=None, seed: int = 0,
                 group=None, fused: bool = False, exchange: str = "chain", dependent: bool = True,
                 panels: bool = True, column_shards: bool = True,
                 weights_from: "LayerStack | None" = None) -> None:
        self.layers, self.batch, self.shape = layers, batch, shape
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device if device is not None else "cuda")
        self.lib = _native.lib()
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed * 1000 + rank)
        self.fused = fused
        self.projections = shape.projections(fused)
        for _, n, _ in self.projections:
            if n % world or (n // world) % 32:
                raise ValueError(f"{n} output rows do not shard evenly over {world} ranks")
        if exchange not in ("chain", "launches"):
            raise ValueError(f"unknown exchange mode {exchange!r}")
        if exchange == "chain" and batch != 1:
            raise ValueError("the chain runs batch 1; use exchange='launches' for larger batches")
        self.exchange = exchange
        self.dependent = dependent and exchange == "chain"
        self.use_panels = panels and exchange == "chain"
        # Column shards (several ranks, dependent chain of the fused layer): o and down keep all their rows and a
        # column range, so that o reads the q rows and down the SiLU*up rows this very rank produced; only the
        # partial sums of o and down cross NVLink (two hand-overs per layer instead of four). q|k|v is then
        # sharded like attention heads: every rank holds a slice of q, of k and of v.
        self.column_shards = bool(column_shards and (world > 1 or column_shards == "always") and self.dependent and fused)
        # weights[l][j]: this rank's rows [rank*N/P, (rank+1)*N/P) of projection j in layer l
        if weights_from is not None:       # a second stack (another batch size) over the same resident weights
            if (weights_from.projections, weights_from.world, weights_from.layers) != (self.projections, world, layers):
                raise ValueError("weights_from must have the same layers, projections and sharding")
            self.weights = weights_from.weights
        else:
            self.weights = [[random_blocks_device(*self.shard_shape(name, n, k, layer), gen, self.device)
                             for name, n, k in self.projections] for layer in range(layers)]
        xg = torch.Generator(device=self.device)
        xg.manual_seed(seed + 7)   # same activations on every rank
        self.inputs = {k: torch.randn((batch, k), generator=xg, device=self.device).to(torch.float16)
                       for k in sorted({k for _, _, k in self.projections})}
        self.vocab = vocab
        if vocab:
            tg = torch.Generator(device=self.device)
            tg.manual_seed(seed * 1000 + 999)          # the table is replicated: same bytes on every rank
            self.table = (weights_from.table if weights_from is not None and weights_from.vocab == vocab
                          else random_blocks_device(vocab, shape.hidden, tg, self.device))
            self.ids = torch.randint(0, vocab, (batch,), generator=xg, device=self.device)
            self.embedded = torch.zeros((batch, shape.hidden), dtype=torch.float16, device=self.device)
        self.launches_per_step = (1 if exchange == "chain" else layers * len(self.projections)) + (1 if vocab else 0)
        self.links_per_step = layers * len(self.projections)
        if exchange == "chain":
            self._setup_chain()
        else:
            # full-width outputs; a rank computes its slice and NCCL gathers the rest
            sizes = sorted({n for _, n, _ in self.projections})
            self.shards = {n: torch.zeros((batch, n // world), dtype=torch.float16, device=self.device) for n in sizes}
            self.outputs = {n: torch.zeros((world, batch, n // world) if world > 1 else (batch, n), dtype=torch.float16,
                                           device=self.device) for n in sizes}
            ws_bytes = max(self.lib.tq1_linear_workspace_bytes(batch, n // world, k) for _, n, k in self.projections)
            self.workspace = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=self.device)
            self.workspace_bytes = ws_bytes

    def column_sharded(self, name: str, layer: int) -> bool:
        """o and down of every layer, except the last down (the step's result stays an ordinary row shard), where a
        rank's column range is a whole number of 512-column chunks; otherwise the projection is sharded by rows."""
        if not self.column_shards or not (name == "o" or (name == "down" and layer != self.layers - 1)):
            return False
        columns = {n_: k_ for n_, _, k_ in self.projections}[name]
        return columns % (512 * self.world) == 0

    def shard_shape(self, name: str, n: int, k: int, layer: int) -> tuple[int, int]:
        """(rows, columns) of this rank's part of a projection."""
        if self.column_sharded(name, layer):
            return n, k // self.world
        return n // self.world, k

    # ------------------------------------------------------------------
    def chain_links(self, layers: "int | None" = None, panels: "bool | None" = None):
        """The step as chain links over this rank's weight shards (see the module docstring). With ``panels`` the
        links stream the chunk-major panel copies of the weights instead of the canonical blocks."""
        from .chain import Link, blocks_to_panels
        panels = self.use_panels if panels is None else panels
        if panels and not hasattr(self, "panels"):
            # a second, permuted copy of every weight (the canonical one stays for the batched kernels and the oracle)
            self.panels = [[blocks_to_panels(w) for w in layer] for layer in self.weights]
        shape, world = self.shape, self.world
        hidden = shape.hidden
        links, outs = [], []
        q_rows = shape.q_heads * shape.head_dim
        # the first layer reads the gathered embedding row; its output scale also brings that row to unit RMS
        x0 = self.embedded[0] if self.vocab else self.inputs[hidden][0]
        x0_gain = self.embedding_gain if self.vocab else 1.0
        for layer in range(self.layers if layers is None else layers):
            blocks = self.weights[layer]
            base = len(links)
            for j, (name, n, k) in enumerate(self.projections):
                swiglu = self.dependent and name == "gate_up"
                partial = self.column_sharded(name, layer)
                rows, k = self.shard_shape(name, n, k, layer)
                n_out = rows // 2 if swiglu else rows
                # a column shard's output is a partial sum: kept in FP32 so that the ranks' parts can be compared
                y = torch.zeros(n_out, dtype=torch.float32 if partial else torch.float16, device=self.device)
                if panels:
                    link = Link(blocks=self.panels[layer][j], panel_rows=rows, y=y, swiglu=swiglu, partial=partial)
                else:
                    link = Link(blocks=blocks[j], y=y, swiglu=swiglu, partial=partial)
                if not self.dependent:
                    link.x = self.inputs[k][0]
                    link.out_scale = unit_gain(k)
                elif name in ("qkv", "q", "k", "v"):
                    link.out_scale = unit_gain(k)
                    if layer == 0:
                        link.x = x0
                        link.out_scale *= x0_gain
                    else:
                        link.source = base - 1                      # the previous layer's down projection
                elif name == "o":
                    link.source, link.source_offset = base, 0       # the q part of q|k|v (or q itself)
                    if partial:                                     # this rank's own q rows: the head of its q|k|v slice
                        link.source_offset = self.rank * (self.projections[0][1] // world)
                    link.out_scale = unit_gain(k * (world if partial else 1))
                    assert q_rows == k * (world if partial else 1)
                elif name in ("gate_up", "gate", "up"):
                    link.source = base + (1 if self.fused else 3)   # the o projection
                    link.out_scale = swiglu_gain(1.0 / unit_gain(k)) if swiglu else unit_gain(k)
                elif name == "down":
                    if self.fused:
                        link.source = base + 2                      # silu(gate) * up
                        if partial:                                 # the rows of it this rank produced
                            link.source_offset = self.rank * k
                    else:
                        link.x = self.inputs[k][0]                  # separate gate and up matrices cannot be fused here
                    link.out_scale = unit_gain(k)
                links.append(link)
                outs.append(y)
        scales = getattr(self, "link_scales", None)          # measured at set-up (see _calibrate)
        if scales is not None and self.dependent:
            for link, scale in zip(links, scales):
                link.out_scale = scale
        return links, outs

    def _calibrate(self, links) -> None:
        """Measured output scales: every link is run once, in order, through the plain entry point on this rank's
        rows, and its scale is set so that the gathered output has unit RMS (the sums of squares are all-reduced,
        so every rank arrives at the same numbers). The analytic gains drift by a fraction of a percent per link,
        which over hundreds of dependent links leaves the FP16 range."""
        import torch.distributed as dist
        from .ops import tq1_matmul
        if self.vocab:          # the gathered row the first link reads
            check(self.lib.tq1_embedding_f16(self.table.data_ptr(), self.ids.data_ptr(), self.embedded.data_ptr(), 0,
                                             self.batch, self.vocab, self.shape.hidden,
                                             ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        gathered = {}
        for i, link in enumerate(links):
            if link.x is not None:
                x = link.x
            else:
                x = gathered[link.source][link.source_offset: link.source_offset + link.columns]
            canonical = self.weights[i // len(self.projections)][i % len(self.projections)]   # the link may stream a permuted copy
            y = tq1_matmul(canonical, x.reshape(1, -1).contiguous(), out_dtype=torch.float32)[0]
            if link.swiglu:
                gate, up = y[0::2], y[1::2]
                y = gate / (1.0 + torch.exp(-gate)) * up
            whole = y
            if link.partial and self.world > 1:             # a column shard: the output is the sum of the ranks' parts
                whole = y.clone()
                dist.all_reduce(whole, group=self.group)
            stats = torch.stack((whole.double().pow(2).sum(),
                                 torch.tensor(float(whole.numel()), dtype=torch.float64, device=y.device)))
            if self.world > 1 and not link.partial:
                dist.all_reduce(stats, group=self.group)
            rms = math.sqrt(float(stats[0] / stats[1]))
            link.out_scale = 1.0 / max(rms, 1e-20)
            if link.partial and self.world > 1:
                # exactly the kernel's arithmetic (scale each part in FP32, add the parts in rank order, round once):
                # SiLU*up makes the chain amplify any difference in scale between this pass and the real step
                parts = torch.empty((self.world, y.numel()), dtype=torch.float32, device=y.device)
                dist.all_gather_into_tensor(parts, (y * link.out_scale).contiguous(), group=self.group)
                total = parts[0].clone()
                for r in range(1, self.world):
                    total += parts[r]
                out = total.to(torch.float16)
            else:
                out = (y * link.out_scale).to(torch.float16)
                if self.world > 1:
                    full = torch.empty((self.world, out.numel()), dtype=out.dtype, device=out.device)
                    dist.all_gather_into_tensor(full, out.contiguous(), group=self.group)
                    out = full.reshape(-1)
            gathered[i] = out
            for j in [j for j in gathered if j < i - 8]:        # sources are never more than a layer back
                del gathered[j]
        torch.cuda.synchronize(self.device)

    def _setup_chain(self) -> None:
        from .chain import ChainPlan
        self.embedding_gain = 1.0 / math.sqrt(0.6 * 0.02 ** 2)      # a decoded embedding row has RMS sqrt(0.6) * 0.02
        links, self.link_outputs = self.chain_links()
        if self.dependent:
            self._calibrate(links)
            self.link_scales = [link.out_scale for link in links]
        peers = None
        if self.world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            from .chain import _pack_links
            nbytes = self.lib.tq1_chain_handoff_bytes(_pack_links(links), len(links), self.world)
            area = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            area.zero_()
            handle = symm_mem.rendezvous(area, self.group if self.group is not None else dist.group.WORLD)
            self._handoff, self._handle = area, handle
            peers = (self.rank, self.world, [int(p) for p in handle.buffer_ptrs])
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        self.plan = ChainPlan(links, peers=peers)
        self.workspace = self.plan.workspace
        self.workspace_bytes = self.workspace.numel()
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------
    @property
    def packed_bytes_per_step(self) -> int:
        """Packed weight bytes this rank streams per step."""
        return self.layers * self.shape.packed_bytes_per_layer() // self.world

    @property
    def algorithmic_bytes_per_step(self) -> int:
        """Packed weights + FP16 activations in + FP16 outputs out, this rank, one step."""
        total = 0
        for layer in range(self.layers):
            for name, n, k in self.projections:
                rows, columns = self.shard_shape(name, n, k, layer)
                total += rows * columns // BLOCK_SIZE * BLOCK_BYTES + 2 * self.batch * (columns + rows)
        if self.vocab:
            total += self.batch * (self.shape.hidden // BLOCK_SIZE * BLOCK_BYTES + 2 * self.shape.hidden)
        return total

    def step(self) -> None:
        """Enqueue one decode step on the current stream (no synchronisation)."""
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        lib, batch, world = self.lib, self.batch, self.world
        if self.vocab:
            check(lib.tq1_embedding_f16(self.table.data_ptr(), self.ids.data_ptr(), self.embedded.data_ptr(),
                                        0, batch, self.vocab, self.shape.hidden, stream))
        if self.exchange == "chain":
            self.plan.run()
            return
        ws, ws_bytes = self.workspace.data_ptr(), self.workspace_bytes
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

    def status(self) -> int:
        """Word 0 of the workspace: non-zero after a bounded device wait ran out (synchronises)."""
        return int(self.workspace[:4].view(torch.int32)[0].item())

    def checksum(self) -> float:
        """Consumes the outputs so the work cannot be dead-coded. In chain mode the last link's output depends on
        every earlier link of every rank."""
        if self.exchange == "chain":
            return float(sum(y.float().abs().sum() for y in self.link_outputs[-len(self.projections):]))
        return float(sum(v.float().abs().sum() for v in self.outputs.values()))
