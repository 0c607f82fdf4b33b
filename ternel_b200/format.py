"""TQ1_G128 block codec with the reference's names and error behaviour.

Mirrors ``bonsai_tq1.format`` of the reference (src/bonsai_tq1/format.py:14-122):
``encode_tq1_blocks`` / ``decode_tq1_blocks`` / ``FormatError`` keep their
argument meaning and messages; the work is done by the native host codec
(``tq1_pack_blocks`` / ``tq1_unpack_blocks`` / ``tq1_validate_blocks``).
"""

from __future__ import annotations

import ctypes

import numpy as np
import numpy.typing as npt

from . import _native

BLOCK_SIZE = 128
BLOCK_BYTES = 28
TRIT_BYTES = 26
MAX_FULL_CODE_BYTE = 3**5 - 1
MAX_TAIL_CODE_BYTE = 3**3 - 1


class FormatError(ValueError):
    """Raised for every shape, dtype or byte-range violation, before any launch."""


def _ptr(array: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(array.ctypes.data)


def check(status: int) -> None:
    """Turn a C-ABI status into the exception the reference raises for it."""
    if status == _native.TQ1_OK:
        return
    message = _native.last_error()
    if status in (_native.TQ1_ERR_INVALID, _native.TQ1_ERR_FORMAT):
        raise FormatError(message)
    raise RuntimeError(f"ternel_b200 native call failed ({status}): {message}")


def encode_tq1_blocks(scales: npt.ArrayLike, codes: npt.ArrayLike) -> np.ndarray:
    """Ternary codes 0/1/2 (+ raw FP16 scale bytes) -> ``(N, 28)`` blocks.

    Same contract as the reference's ``encode_tq1_blocks`` (format.py:66-91).
    """
    scale_array = np.ascontiguousarray(scales, dtype=np.uint8)
    code_array = np.ascontiguousarray(codes, dtype=np.uint8)
    if scale_array.ndim == 1:
        scale_array = scale_array.reshape(-1, 2)
    if code_array.ndim == 1:
        code_array = code_array.reshape(-1, BLOCK_SIZE)
    if scale_array.ndim != 2 or scale_array.shape[1] != 2:
        raise FormatError(f"expected scale bytes shaped (N, 2), got {scale_array.shape}")
    if code_array.ndim != 2 or code_array.shape[1] != BLOCK_SIZE:
        raise FormatError(f"expected codes shaped (N, 128), got {code_array.shape}")
    if scale_array.shape[0] != code_array.shape[0]:
        raise FormatError("scale and code block counts differ")
    count = code_array.shape[0]
    out = np.empty((count, BLOCK_BYTES), dtype=np.uint8)
    bad = ctypes.c_int64(0)
    check(_native.lib().tq1_pack_blocks(_ptr(scale_array), _ptr(code_array), _ptr(out), count,
                                        ctypes.byref(bad)))
    return out


def _as_blocks(blocks: npt.ArrayLike) -> np.ndarray:
    packed = np.ascontiguousarray(blocks, dtype=np.uint8)
    if packed.ndim == 1:
        if packed.size % BLOCK_BYTES:
            raise FormatError("TQ1 byte length is not divisible by 28")
        packed = packed.reshape(-1, BLOCK_BYTES)
    if packed.ndim != 2 or packed.shape[1] != BLOCK_BYTES:
        raise FormatError(f"expected TQ1 blocks shaped (N, 28), got {packed.shape}")
    return packed


def decode_tq1_blocks(blocks: npt.ArrayLike, *, validate: bool = True) -> tuple[np.ndarray, np.ndarray]:
    """``(N, 28)`` blocks -> ``(scale bytes (N,2), codes (N,128))`` (format.py:94-122)."""
    packed = _as_blocks(blocks)
    count = packed.shape[0]
    scales = np.empty((count, 2), dtype=np.uint8)
    codes = np.empty((count, BLOCK_SIZE), dtype=np.uint8)
    bad_full, bad_tail = ctypes.c_int64(0), ctypes.c_int64(0)
    check(_native.lib().tq1_unpack_blocks(_ptr(packed), _ptr(scales), _ptr(codes), count,
                                          int(bool(validate)), ctypes.byref(bad_full),
                                          ctypes.byref(bad_tail)))
    return scales, codes


def dequantize_blocks(blocks: npt.ArrayLike) -> np.ndarray:
    """``(N, 28)`` blocks -> FP32 weights ``(N, 128)``, ``(trit - 1) * scale`` (the host-side ``to_float`` of the
    type, ``dequantize_row_tq1_g128``, patches/prism-tq1-g128-distribution.patch:423-440)."""
    packed = _as_blocks(blocks)
    out = np.empty((packed.shape[0], BLOCK_SIZE), dtype=np.float32)
    check(_native.lib().tq1_dequantize_blocks(_ptr(packed), _ptr(out), packed.shape[0]))
    return out


def validate_blocks(blocks: npt.ArrayLike) -> None:
    """Fail-closed scan of canonical blocks for bytes > 242 (full) / > 26 (tail)."""
    packed = _as_blocks(np.asarray(blocks).reshape(-1, BLOCK_BYTES) if np.asarray(blocks).ndim > 2 else blocks)
    bad_full, bad_tail = ctypes.c_int64(0), ctypes.c_int64(0)
    check(_native.lib().tq1_validate_blocks(_ptr(packed), packed.shape[0], ctypes.byref(bad_full),
                                            ctypes.byref(bad_tail)))
