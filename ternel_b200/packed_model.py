"""Swap the linear and embedding leaves of a built torch model for their packed equivalents.

The torch-side counterpart of the reference's graph surgery
(src/ternel_mlx/packed_model.py:72-92, ``replace_with_packed``): walk the module
tree, replace every ``nn.Linear`` by a ``PackedLinear`` of the same shape and
every ``nn.Embedding`` by a ``PackedEmbedding``, and return a count per kind so
that the caller can assert that the graph it got is the graph it expected
(src/ternel_mlx/packed_model.py:108-117). The packed modules start as all-zero
matrices; a converted checkpoint's ``<path>.codes`` / ``<path>.scales`` (or
``<path>.blocks``) arrays are then installed with ``load_state_dict``.
"""

from __future__ import annotations

from collections.abc import Iterable

import numpy as np
import torch
from torch import nn

from .format import FormatError, encode_tq1_blocks
from .modules import PackedEmbedding, PackedLinear


def replace_with_packed(model: nn.Module, *, dtype: torch.dtype = torch.float16, device=None,
                        skip: Iterable[str] = ()) -> dict[str, int]:
    """Replace, in place, every ``nn.Linear`` / ``nn.Embedding`` below ``model``.

    ``skip`` names module paths (as in ``named_modules``) to leave dense. A linear
    layer with a bias raises ``FormatError``, as in the reference
    (src/ternel_mlx/modules.py:483-484). Returns ``{"linear": n, "embedding": m}``.
    """
    counts = {"linear": 0, "embedding": 0}
    skipped = set(skip)

    def walk(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            path = f"{prefix}.{name}" if prefix else name
            if path in skipped:
                continue
            if isinstance(child, nn.Linear):
                setattr(parent, name, PackedLinear.from_linear(child, device=device))
                counts["linear"] += 1
            elif isinstance(child, nn.Embedding):
                setattr(parent, name, PackedEmbedding.from_embedding(child, dtype=dtype, device=device))
                counts["embedding"] += 1
            else:
                walk(child, path)

    walk(model, "")
    return counts


def expect_counts(counts: dict[str, int], *, embeddings: int = 1, min_linear: int = 1) -> None:
    """The reference's sanity check after the swap (src/ternel_mlx/packed_model.py:108-117)."""
    if counts["embedding"] != embeddings:
        raise FormatError(f"expected exactly {embeddings} embedding table(s), replaced {counts['embedding']}")
    if counts["linear"] < min_linear:
        raise FormatError("no linear layers were replaced; the graph is not what was expected")


def blocks_from_ternary(trits: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """Canonical blocks ``[rows][columns/128][28]`` from weights given as trits in {-1, 0, +1}
    (``[rows, columns]``) and one FP16 scale per 128-group (``[rows, columns/128]``)."""
    trits = np.asarray(trits)
    rows, columns = trits.shape
    if columns % 128:
        raise FormatError(f"{columns} columns is not a multiple of the 128-weight group")
    scales = np.asarray(scales, dtype=np.float16)
    if scales.shape != (rows, columns // 128):
        raise FormatError(f"expected scales of shape {(rows, columns // 128)}, got {scales.shape}")
    if trits.min(initial=0) < -1 or trits.max(initial=0) > 1:
        raise FormatError("weights must be -1, 0 or +1")
    codes = (trits.astype(np.int16) + 1).astype(np.uint8).reshape(-1, 128)
    raw = scales.reshape(-1).view(np.uint8).reshape(-1, 2)
    return encode_tq1_blocks(raw, codes).reshape(rows, columns // 128, 28)


def dense_from_ternary(trits: np.ndarray, scales: np.ndarray) -> torch.Tensor:
    """The dense FP32 matrix the packed one stands for (for building a dense twin in tests)."""
    trits = np.asarray(trits, dtype=np.float32)
    s = np.repeat(np.asarray(scales, dtype=np.float16).astype(np.float32), 128, axis=1)
    return torch.from_numpy(trits * s)
