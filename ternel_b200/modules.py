"""``nn.Module`` drop-ins for a converted model's linear and embedding leaves.

``PackedLinear`` / ``PackedEmbedding`` / ``packed_matmul`` keep the surface of
the reference's modules (src/ternel_mlx/modules.py:425-549): bias-free, any
leading dimensions, last dimension checked before any launch, output in the
activation dtype, out-of-range token ids giving zero rows, and a tied-head
``as_linear``. The weight lives on the GPU as canonical 28-byte blocks for the
module's whole life; nothing is ever dequantised into a dense matrix.

A converted checkpoint names two arrays per packed module, ``<path>.codes``
(uint8 ``[tiles, groups, 26, tile]``) and ``<path>.scales`` (uint16
``[tiles, groups, tile]``) (src/ternel_mlx/layout.py:36-38); ``load_state_dict``
accepts that pair as well as this library's own ``<path>.blocks`` and rejects
missing or mis-shaped arrays and out-of-range code bytes (fail closed).
"""

from __future__ import annotations

import numpy as np
import torch
from torch import nn

from .format import BLOCK_BYTES, FormatError, validate_blocks
from .layout import CODES_SUFFIX, SCALES_SUFFIX, PackedTensorLayout, unpack_blocks, validate_packed_codes
from .ops import tq1_get_rows, tq1_matmul, validate_device_blocks


def packed_matmul(blocks: torch.Tensor, x: torch.Tensor, *, layout: PackedTensorLayout,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ W.T`` for packed ``W`` with any leading dimensions on ``x``."""
    if x.shape[-1] != layout.columns:
        raise FormatError(
            f"activation has {x.shape[-1]} columns, weight expects {layout.columns}")
    flat = x.reshape(-1, layout.columns)
    out = tq1_matmul(blocks, flat, out_dtype=out_dtype)
    return out.reshape(*x.shape[:-1], layout.rows)


class _PackedBase(nn.Module):
    layout: PackedTensorLayout

    def __init__(self, layout: PackedTensorLayout, device=None) -> None:
        super().__init__()
        self.layout = layout
        self.register_buffer("blocks", torch.zeros(layout.blocks_shape, dtype=torch.uint8, device=device))
        # zero bytes decode to code 0 = weight -1 with scale +0.0, i.e. an all-zero matrix
        self._validated = False

    # -- loading ----------------------------------------------------------
    def load_blocks(self, blocks, *, validate: bool = True) -> None:
        """Install canonical blocks (NumPy or tensor) after the fail-closed byte scan."""
        if isinstance(blocks, torch.Tensor):
            tensor = blocks
        else:
            array = np.ascontiguousarray(blocks)
            if array.dtype != np.uint8:
                raise FormatError(f"canonical blocks must be uint8, got {array.dtype}")
            tensor = torch.from_numpy(array)
        if tensor.dtype != torch.uint8:
            raise FormatError(f"canonical blocks must be uint8, got {tensor.dtype}")
        if tuple(tensor.shape) != self.layout.blocks_shape:
            raise FormatError(
                f"expected canonical blocks of shape {self.layout.blocks_shape}, got {tuple(tensor.shape)}")
        if validate:
            if tensor.is_cuda:
                validate_device_blocks(tensor.contiguous())
            else:
                validate_blocks(tensor.contiguous().numpy().reshape(-1, BLOCK_BYTES))
        self.blocks.copy_(tensor)
        self._validated = validate

    def load_tiled(self, codes, scales) -> None:
        """Install the reference's tiled ``codes`` / ``scales`` pair."""
        code_array = codes.cpu().numpy() if isinstance(codes, torch.Tensor) else np.asarray(codes)
        scale_array = scales.cpu().numpy() if isinstance(scales, torch.Tensor) else np.asarray(scales)
        if scale_array.dtype == np.int16:      # torch has no first-class uint16 storage
            scale_array = scale_array.view(np.uint16)
        validate_packed_codes(code_array)
        blocks = unpack_blocks(code_array, scale_array.astype("<u2", copy=False), layout=self.layout)
        self.load_blocks(blocks, validate=False)
        self._validated = True

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        codes_key, scales_key = prefix + CODES_SUFFIX, prefix + SCALES_SUFFIX
        if codes_key in state_dict or scales_key in state_dict:
            if codes_key not in state_dict or scales_key not in state_dict:
                missing_keys.append(scales_key if codes_key in state_dict else codes_key)
                return
            try:
                self.load_tiled(state_dict[codes_key], state_dict[scales_key])
            except FormatError as exc:
                error_msgs.append(f"{prefix.rstrip('.')}: {exc}")
            return
        key = prefix + "blocks"
        if key not in state_dict:
            if strict:
                missing_keys.append(key)
            return
        try:
            self.load_blocks(state_dict[key])
        except FormatError as exc:
            error_msgs.append(f"{prefix.rstrip('.')}: {exc}")


class PackedLinear(_PackedBase):
    """A bias-free linear layer whose weight stays in TQ1_G128 for its lifetime."""

    def __init__(self, layout: PackedTensorLayout, device=None, out_dtype: torch.dtype | None = None) -> None:
        super().__init__(layout, device=device)
        self.out_dtype = out_dtype

    @classmethod
    def from_linear(cls, linear: nn.Linear, device=None) -> "PackedLinear":
        """Take the shape from a built ``nn.Linear``; its dense weight is not used."""
        if linear.bias is not None:
            raise FormatError("a packed linear layer cannot carry a bias")
        rows, columns = linear.weight.shape
        return cls(PackedTensorLayout.for_tensor(rows, columns),
                   device=device if device is not None else linear.weight.device)

    def extra_repr(self) -> str:
        return (f"{self.layout.columns} -> {self.layout.rows}, "
                f"{self.layout.bits_per_weight:.3f} bits/weight")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return packed_matmul(self.blocks, x, layout=self.layout, out_dtype=self.out_dtype)


class PackedEmbedding(_PackedBase):
    """A token embedding decoded one row at a time straight out of the packed bytes."""

    def __init__(self, layout: PackedTensorLayout, *, dtype: torch.dtype = torch.float16, device=None) -> None:
        super().__init__(layout, device=device)
        self.dtype = dtype

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding, *, dtype: torch.dtype = torch.float16,
                       device=None) -> "PackedEmbedding":
        rows, columns = embedding.weight.shape
        return cls(PackedTensorLayout.for_tensor(rows, columns), dtype=dtype,
                   device=device if device is not None else embedding.weight.device)

    def extra_repr(self) -> str:
        return f"{self.layout.rows} x {self.layout.columns}, {self.dtype}"

    def forward(self, indices: torch.Tensor) -> torch.Tensor:
        """Gather rows for ``indices`` of any shape and integer dtype, as ``nn.Embedding`` does."""
        flat = indices.reshape(-1)
        rows = tq1_get_rows(self.blocks, flat, dtype=self.dtype)
        return rows.reshape(*indices.shape, self.layout.columns)

    def as_linear(self, x: torch.Tensor) -> torch.Tensor:
        """The tied-output-head path: the embedding table used as a matmul."""
        return packed_matmul(self.blocks, x, layout=self.layout)
