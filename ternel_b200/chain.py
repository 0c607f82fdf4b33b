"""Chains of batch-1 packed products that run as one persistent kernel launch.

A decoded token issues one matrix-vector product per packed linear, back to back
(the reference's converted model calls ``packed_matmul`` for every linear leaf of
every layer, src/ternel_mlx/modules.py:425-457,460-495). ``ChainPlan`` describes such
a sequence once and replays it with a single launch of ``tq1_gemv_chain_kernel``: a
link either reads FP16 activations that exist before the launch or the output of an
earlier link of the same chain, and may apply ``silu(gate) * up`` over (gate, up) row
pairs and an output scale in its epilogue.

With ``peers`` the rows of every link are sharded over the ranks of a process group
and finished outputs are pushed into every rank's hand-off area (symmetric memory).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _native
from .format import BLOCK_BYTES, BLOCK_SIZE, FormatError, check


@dataclass
class Link:
    """One product of a chain. ``blocks``: canonical ``uint8[N, K/128, 28]`` on the GPU (this rank's rows).

    ``x``: FP16 ``[K]`` tensor complete before the launch, or ``None`` to read the output of link
    ``source`` (an earlier link) starting at element ``source_offset``. ``y``: optional output tensor
    (FP16 or FP32, ``N`` elements, ``N/2`` with ``swiglu``). With ``panel_rows > 0`` ``blocks`` holds the
    chunk-major panel form of ``blocks_to_panels`` for a weight of that many rows. ``partial`` (sharded
    chains): this rank holds a column range of the matrix, its output is a partial sum, and a link that
    reads it receives the ranks' sum (see ``tq1_chain_peers`` in the header).
    """

    blocks: torch.Tensor
    x: torch.Tensor | None = None
    source: int = -1
    source_offset: int = 0
    y: torch.Tensor | None = None
    swiglu: bool = False
    out_scale: float = 1.0
    panel_rows: int = 0
    partial: bool = False

    @property
    def rows(self) -> int:
        return self.panel_rows if self.panel_rows else self.blocks.shape[0]

    @property
    def columns(self) -> int:
        return self.blocks.shape[0] * 512 if self.panel_rows else self.blocks.shape[1] * BLOCK_SIZE

    @property
    def outputs(self) -> int:
        return self.rows // 2 if self.swiglu else self.rows


def _pack_links(links: list[Link]):
    array = (_native.ChainLink * len(links))()
    for i, link in enumerate(links):
        b = link.blocks
        if link.panel_rows:
            pad = (link.panel_rows + 15) // 16 * 16
            if b.dtype != torch.uint8 or b.dim() != 3 or b.shape[1] != pad or b.shape[2] != 112 or not b.is_contiguous():
                raise FormatError(f"link {i}: panels of {link.panel_rows} rows must be contiguous uint8 "
                                  f"(chunks, {pad}, 112), got {tuple(b.shape)}")
        elif b.dtype != torch.uint8 or b.dim() != 3 or b.shape[2] != BLOCK_BYTES or not b.is_contiguous():
            raise FormatError(f"link {i}: blocks must be contiguous uint8 (rows, groups, 28), got {tuple(b.shape)}")
        if not b.is_cuda:
            raise RuntimeError(f"link {i}: blocks are on {b.device}; the packed ternary kernels run on CUDA only")
        c = array[i]
        c.blocks, c.N, c.K = b.data_ptr(), link.rows, link.columns
        if link.x is not None:
            if link.x.dtype != torch.float16 or link.x.numel() != link.columns or not link.x.is_contiguous():
                raise FormatError(f"link {i}: x must be contiguous FP16 with {link.columns} elements")
            c.x, c.source = link.x.data_ptr(), -1
        else:
            if not 0 <= link.source < i:
                raise FormatError(f"link {i}: source {link.source} is not an earlier link")
            c.x, c.source = None, link.source
        c.source_offset = link.source_offset
        if link.y is not None:
            if link.y.dtype not in (torch.float16, torch.float32) or link.y.numel() != link.outputs \
                    or not link.y.is_contiguous():
                raise FormatError(f"link {i}: y must be contiguous FP16/FP32 with {link.outputs} elements")
            c.y, c.y_is_f32 = link.y.data_ptr(), int(link.y.dtype == torch.float32)
        else:
            c.y, c.y_is_f32 = None, 0
        c.swiglu, c.out_scale = int(link.swiglu), float(link.out_scale)
        c.layout = 1 if link.panel_rows else 0
        c.partial = int(link.partial)
    return array


def blocks_to_panels(blocks: torch.Tensor) -> torch.Tensor:
    """Canonical ``uint8[N, K/128, 28]`` on the GPU -> chunk-major panels ``uint8[K/512, pad16(N), 112]`` (a
    lossless permutation, rows padded with zero blocks): the layout the chain streams fastest."""
    if blocks.dtype != torch.uint8 or blocks.dim() != 3 or blocks.shape[2] != BLOCK_BYTES or not blocks.is_contiguous():
        raise FormatError(f"blocks must be contiguous uint8 (rows, groups, 28), got {tuple(blocks.shape)}")
    if not blocks.is_cuda:
        raise RuntimeError(f"blocks are on {blocks.device}; the packed ternary kernels run on CUDA only")
    rows, columns = blocks.shape[0], blocks.shape[1] * BLOCK_SIZE
    if columns % 512:
        raise FormatError(f"{columns} columns is not a multiple of 512")
    out = torch.empty((columns // 512, (rows + 15) // 16 * 16, 112), dtype=torch.uint8, device=blocks.device)
    with torch.cuda.device(blocks.device):
        check(_native.lib().tq1_blocks_to_panels_device(
            blocks.data_ptr(), out.data_ptr(), rows, columns,
            ctypes.c_void_p(torch.cuda.current_stream(blocks.device).cuda_stream)))
    return out


def panels_to_blocks(panels: torch.Tensor, rows: int) -> torch.Tensor:
    """The inverse of ``blocks_to_panels``: the canonical blocks, byte for byte."""
    if panels.dtype != torch.uint8 or panels.dim() != 3 or panels.shape[2] != 112 or not panels.is_contiguous() \
            or panels.shape[1] != (rows + 15) // 16 * 16:
        raise FormatError(f"panels of {rows} rows must be contiguous uint8 (chunks, pad16(rows), 112), got {tuple(panels.shape)}")
    columns = panels.shape[0] * 512
    out = torch.empty((rows, columns // BLOCK_SIZE, BLOCK_BYTES), dtype=torch.uint8, device=panels.device)
    with torch.cuda.device(panels.device):
        check(_native.lib().tq1_panels_to_blocks_device(
            panels.data_ptr(), out.data_ptr(), rows, columns,
            ctypes.c_void_p(torch.cuda.current_stream(panels.device).cuda_stream)))
    return out


def linear_chain(links: list[Link], workspace: torch.Tensor) -> None:
    """Run up to 8 links as one launch on the current stream (single GPU). ``workspace``: zero-filled once,
    at least ``chain_workspace_bytes(links)`` bytes of uint8 on the GPU."""
    lib = _native.lib()
    array = _pack_links(links)
    device = links[0].blocks.device
    with torch.cuda.device(device):
        check(lib.tq1_linear_chain_f16(array, len(links), workspace.data_ptr(), workspace.numel(),
                                       ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)))


def chain_workspace_bytes(links: list[Link], world: int = 1) -> int:
    return _native.lib().tq1_chain_workspace_bytes(_pack_links(links), len(links), world)


class ChainPlan:
    """A described chain: ``run()`` enqueues one launch on the current stream.

    Owns its workspace and link table (torch tensors); keeps references to the tensors the links
    name, whose addresses the plan has captured.
    """

    def __init__(self, links: list[Link], *, peers: "tuple[int, int, list[int]] | None" = None,
                 workspace: torch.Tensor | None = None) -> None:
        if not links:
            raise FormatError("a chain needs at least one link")
        self.lib = _native.lib()
        self.links = list(links)
        self.device = links[0].blocks.device
        self._array = _pack_links(self.links)
        world = peers[1] if peers else 1
        need = self.lib.tq1_chain_workspace_bytes(self._array, len(links), world)
        if workspace is None:
            workspace = torch.zeros(need, dtype=torch.uint8, device=self.device)
        elif workspace.numel() < need:
            raise FormatError(f"chain workspace of {need} bytes required, got {workspace.numel()}")
        self.workspace = workspace
        table_bytes = self.lib.tq1_chain_table_bytes(self._array, len(links))
        self.table = torch.zeros(max(table_bytes, 256), dtype=torch.uint8, device=self.device)
        peers_struct = None
        if peers:
            peers_struct = _native.ChainPeers()
            peers_struct.rank, peers_struct.world = peers[0], peers[1]
            for r, ptr in enumerate(peers[2]):
                peers_struct.handoff[r] = ptr
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(self.lib.tq1_chain_plan_create(
                self._array, len(links), ctypes.byref(peers_struct) if peers_struct is not None else None,
                self.workspace.data_ptr(), self.workspace.numel(), self.table.data_ptr(), self.table.numel(),
                ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream), ctypes.byref(handle)))
        self._handle = handle

    def run(self) -> None:
        with torch.cuda.device(self.device):
            check(self.lib.tq1_chain_plan_run(self._handle,
                                              ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))

    def status(self) -> int:
        """Word 0 of the workspace: non-zero after a bounded device wait ran out (synchronises)."""
        return int(self.workspace[:4].view(torch.int32)[0].item())

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self.lib.tq1_chain_plan_destroy(self._handle)
            self._handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass
