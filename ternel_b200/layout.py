"""Layout descriptor and the bridge to the reference's tiled arrays.

``PackedTensorLayout`` keeps the reference's shape and byte accounting
(src/ternel_mlx/layout.py:41-147); ``pack_blocks`` / ``unpack_blocks`` /
``validate_packed_codes`` keep the contract of src/ternel_mlx/packing.py:29-82.
On the device this library stores the *canonical* row-major blocks; the tiled
``codes``/``scales`` pair is only an interchange form accepted at load time.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _native
from .format import BLOCK_BYTES, BLOCK_SIZE, MAX_FULL_CODE_BYTE, MAX_TAIL_CODE_BYTE, FormatError, check

PREFERRED_TILE = 256
CODE_SLOTS = 26
FULL_CODE_SLOTS = 25
SCALE_BYTES = BLOCK_BYTES - CODE_SLOTS
SCALE_VIEW_DTYPE = np.dtype("<u2")
CODES_SUFFIX = "codes"
SCALES_SUFFIX = "scales"
PANEL_COLUMNS = 512          # one panel covers this many input columns (four groups = 112 bytes per row)
PANEL_ROW_QUANTUM = 16       # panels are zero-padded to whole 16-row tiles


def select_tile(rows: int) -> int:
    """Row tile of the tiled interchange arrays: the reference tiles by 256 rows and, because it never pads,
    falls back to one tile of all rows when 256 does not divide them (src/ternel_mlx/layout.py:41-51)."""
    if rows <= 0:
        raise FormatError(f"row count must be positive, got {rows}")
    whole_tiles, leftover = divmod(rows, PREFERRED_TILE)
    return PREFERRED_TILE if whole_tiles and not leftover else rows


@dataclass(frozen=True)
class PackedTensorLayout:
    """Where the bytes of one packed weight ``W[rows out][columns in]`` live, in each of the three forms this
    library handles:

    * canonical blocks ``uint8[rows][columns/128][28]`` -- what the C ABI takes and every kernel can read;
    * chunk-major panels ``uint8[columns/512][pad16(rows)][112]`` -- the streaming form of the batch-1 chain
      (only when ``columns`` is a multiple of 512);
    * the reference's tiled pair ``codes uint8[tiles][groups][26][tile]`` + ``scales uint16[tiles][groups][tile]``
      (src/ternel_mlx/layout.py:54-147), accepted at load time and converted; ``tile`` only describes this form.

    All three hold the same 28 bytes per 128 weights, so one byte count serves them (panels add zero rows).
    """

    rows: int
    columns: int
    tile: int

    def __post_init__(self) -> None:
        for name, value in (("rows", self.rows), ("columns", self.columns), ("tile", self.tile)):
            if value <= 0:
                what = "tile must be positive" if name == "tile" else "tensor dimensions must be positive"
                raise FormatError(f"{what}, got {self.rows}x{self.columns} with tile {self.tile}")
        if self.columns % BLOCK_SIZE:
            raise FormatError(f"{self.columns} columns is not a multiple of the {BLOCK_SIZE}-weight group")
        if self.rows % self.tile:
            raise FormatError(f"tile {self.tile} does not divide {self.rows} rows; the layout does not pad rows")

    @classmethod
    def for_tensor(cls, rows: int, columns: int) -> "PackedTensorLayout":
        return cls(rows=rows, columns=columns, tile=select_tile(rows))

    # ---- counts -----------------------------------------------------------------------------------------
    @property
    def groups_per_row(self) -> int:
        return self.columns // BLOCK_SIZE

    @property
    def groups(self) -> int:
        """128-weight groups (= 28-byte blocks) in the whole tensor."""
        return self.rows * self.groups_per_row

    @property
    def tiles(self) -> int:
        return self.rows // self.tile

    # ---- canonical blocks and panels (device forms) --------------------------------------------------------
    @property
    def blocks_shape(self) -> tuple[int, int, int]:
        return (self.rows, self.groups_per_row, BLOCK_BYTES)

    @property
    def canonical_bytes(self) -> int:
        return self.groups * BLOCK_BYTES

    @property
    def streams_as_panels(self) -> bool:
        return self.columns % PANEL_COLUMNS == 0

    @property
    def panels_shape(self) -> tuple[int, int, int]:
        if not self.streams_as_panels:
            raise FormatError(f"{self.columns} columns is not a multiple of {PANEL_COLUMNS}: no panel form")
        padded = -(-self.rows // PANEL_ROW_QUANTUM) * PANEL_ROW_QUANTUM
        return (self.columns // PANEL_COLUMNS, padded, PANEL_COLUMNS // BLOCK_SIZE * BLOCK_BYTES)

    @property
    def panel_bytes(self) -> int:
        chunks, padded, row_bytes = self.panels_shape
        return chunks * padded * row_bytes

    # ---- the reference's tiled interchange form -------------------------------------------------------------
    @property
    def codes_shape(self) -> tuple[int, int, int, int]:
        return (self.tiles, self.groups_per_row, CODE_SLOTS, self.tile)

    @property
    def scales_shape(self) -> tuple[int, int, int]:
        return (self.tiles, self.groups_per_row, self.tile)

    @property
    def codes_bytes(self) -> int:
        return self.groups * CODE_SLOTS

    @property
    def scales_bytes(self) -> int:
        return self.groups * SCALE_BYTES

    @property
    def payload_bytes(self) -> int:
        """Bytes of the tiled pair; always ``canonical_bytes`` (26 code bytes + 2 scale bytes per group)."""
        return self.codes_bytes + self.scales_bytes

    @property
    def bits_per_weight(self) -> float:
        return 8.0 * BLOCK_BYTES / BLOCK_SIZE


def validate_packed_codes(codes: np.ndarray) -> None:
    """Reject any tiled code byte above 242 (full slots) or 26 (tail slot)."""
    array = np.asarray(codes)
    if array.dtype != np.uint8:
        raise FormatError(f"codes must be uint8, got {array.dtype}")
    if array.ndim != 4:
        raise FormatError(f"codes must be 4-D (tiles, groups, slots, tile), got {array.shape}")
    invalid_full = int(np.count_nonzero(array[:, :, :FULL_CODE_SLOTS, :] > MAX_FULL_CODE_BYTE))
    invalid_tail = int(np.count_nonzero(array[:, :, FULL_CODE_SLOTS, :] > MAX_TAIL_CODE_BYTE))
    if invalid_full or invalid_tail:
        raise FormatError(
            f"packed codes contain out-of-range base-3 bytes: regular={invalid_full} "
            f"(max {MAX_FULL_CODE_BYTE}), tail={invalid_tail} (max {MAX_TAIL_CODE_BYTE})")


def _ptr(array: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(array.ctypes.data)


def pack_blocks(blocks: np.ndarray, *, layout: PackedTensorLayout) -> tuple[np.ndarray, np.ndarray]:
    """Canonical ``(rows, groups, 28)`` -> tiled ``(codes uint8, scales uint16)``."""
    source = np.asarray(blocks)
    if source.dtype != np.uint8:
        raise FormatError(f"canonical blocks must be uint8, got {source.dtype}")
    if source.shape != layout.blocks_shape:
        raise FormatError(f"expected canonical blocks of shape {layout.blocks_shape}, got {source.shape}")
    source = np.ascontiguousarray(source)
    codes = np.empty(layout.codes_shape, dtype=np.uint8)
    scales = np.empty(layout.scales_shape, dtype=SCALE_VIEW_DTYPE)
    check(_native.lib().tq1_tile_blocks(_ptr(source), _ptr(codes), _ptr(scales), layout.rows,
                                        layout.groups_per_row, layout.tile))
    return codes, scales


def unpack_blocks(codes: np.ndarray, scales: np.ndarray, *, layout: PackedTensorLayout) -> np.ndarray:
    """Inverse of :func:`pack_blocks`."""
    code_array = np.asarray(codes)
    scale_array = np.asarray(scales)
    if code_array.dtype != np.uint8:
        raise FormatError(f"codes must be uint8, got {code_array.dtype}")
    if scale_array.dtype != SCALE_VIEW_DTYPE:
        raise FormatError(f"scales must be little-endian uint16, got {scale_array.dtype}")
    if code_array.shape != layout.codes_shape:
        raise FormatError(f"codes shape {code_array.shape} does not match {layout.codes_shape}")
    if scale_array.shape != layout.scales_shape:
        raise FormatError(f"scales shape {scale_array.shape} does not match {layout.scales_shape}")
    code_array = np.ascontiguousarray(code_array)
    scale_array = np.ascontiguousarray(scale_array)
    blocks = np.empty(layout.blocks_shape, dtype=np.uint8)
    check(_native.lib().tq1_untile_blocks(_ptr(code_array), _ptr(scale_array), _ptr(blocks),
                                          layout.rows, layout.groups_per_row, layout.tile))
    return blocks


@dataclass(frozen=True)
class ModelLinearShape:
    """One distinct linear weight shape of the 27B model and how many matmuls of that shape one decoded token
    issues. The reference keeps the same census for its benchmarks (src/ternel_mlx/layout.py:150-198); here the
    counts are derived from the layer structure so that the arithmetic is visible."""

    label: str
    rows: int
    columns: int
    dispatches_per_token: int

    def layout(self) -> PackedTensorLayout:
        return PackedTensorLayout.for_tensor(self.rows, self.columns)


# The model interleaves 48 linear-attention layers with 16 full-attention layers; every layer has a gated MLP.
# Shapes outside the four benchmark shapes matter for coverage: 48 rows (not a multiple of 16 x 8 or of the
# 256-row tile), K = 6144, and a 248,320-row head.
_LINEAR_ATTN_LAYERS, _FULL_ATTN_LAYERS = 48, 16
_ALL_LAYERS = _LINEAR_ATTN_LAYERS + _FULL_ATTN_LAYERS
MODEL_LINEAR_SHAPES: tuple[ModelLinearShape, ...] = (
    ModelLinearShape("linear_attn.in_proj_a/b", 48, 5120, 2 * _LINEAR_ATTN_LAYERS),
    ModelLinearShape("self_attn.k_proj/v_proj", 1024, 5120, 2 * _FULL_ATTN_LAYERS),
    ModelLinearShape("linear_attn.out_proj, self_attn.o_proj", 5120, 6144, _ALL_LAYERS),
    ModelLinearShape("mlp.down_proj", 5120, 17408, _ALL_LAYERS),
    ModelLinearShape("linear_attn.in_proj_z", 6144, 5120, _LINEAR_ATTN_LAYERS),
    ModelLinearShape("linear_attn.in_proj_qkv", 10240, 5120, _LINEAR_ATTN_LAYERS),
    ModelLinearShape("self_attn.q_proj", 12288, 5120, _FULL_ATTN_LAYERS),
    ModelLinearShape("mlp.gate_proj/up_proj", 17408, 5120, 2 * _ALL_LAYERS),
    ModelLinearShape("lm_head", 248320, 5120, 1),
)
# eight matmuls per linear-attention layer, seven per full-attention layer, one output head
DISPATCHES_PER_TOKEN = 8 * _LINEAR_ATTN_LAYERS + 7 * _FULL_ATTN_LAYERS + 1
if sum(shape.dispatches_per_token for shape in MODEL_LINEAR_SHAPES) != DISPATCHES_PER_TOKEN:
    raise FormatError("the shape census no longer accounts for a whole decoded token")
