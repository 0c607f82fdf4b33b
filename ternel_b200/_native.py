"""ctypes binding of the C ABI declared in include/ternel_b200.h.

There is no fallback: if the shared library is missing the import of any
compute entry point raises, so a run can never silently continue on a CPU or
PyTorch path.
"""

from __future__ import annotations

import ctypes
import os
from pathlib import Path
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, POINTER

from .build import LIB_PATH

TQ1_OK = 0
TQ1_ERR_INVALID = -1
TQ1_ERR_FORMAT = -2
TQ1_ERR_CUDA = -3
TQ1_ERR_WORKSPACE = -4

# name -> (restype, argtypes); must list every symbol the header declares.
SIGNATURES = {
    "tq1_abi_version": (c_int, []),
    "tq1_last_error": (c_char_p, []),
    "tq1_pack_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, POINTER(c_int64)]),
    "tq1_unpack_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                  POINTER(c_int64), POINTER(c_int64)]),
    "tq1_dequantize_blocks": (c_int, [c_void_p, c_void_p, c_int64]),
    "tq1_validate_blocks": (c_int, [c_void_p, c_int64, POINTER(c_int64), POINTER(c_int64)]),
    "tq1_tile_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "tq1_untile_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]),
    "tq1_validate_blocks_device": (c_int, [c_void_p, c_int64, c_void_p, c_void_p]),
    "tq1_linear_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tq1_linear_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                               c_void_p, c_size_t, c_void_p]),
    "tq1_linear_swiglu_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_void_p, c_size_t, c_void_p]),
    "tq1_linear_plan": (c_int, [c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int),
                                POINTER(c_int)]),
    "tq1_linear_sharded_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "tq1_shard_advance_epoch": (c_int, [c_void_p, ctypes.c_uint32, c_void_p]),
    "tq1_linear_f16_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t,
                                       c_void_p]),
    "tq1_gemv_f16_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "tq1_gemv_noalloc_status": (c_int, [c_void_p, c_void_p]),
    "tq1_panel_bytes": (c_size_t, [c_int, c_int]),
    "tq1_blocks_to_panels_device": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "tq1_panels_to_blocks_device": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
    "tq1_chain_workspace_bytes": (c_size_t, [c_void_p, c_int, c_int]),
    "tq1_chain_handoff_bytes": (c_size_t, [c_void_p, c_int, c_int]),
    "tq1_chain_table_bytes": (c_size_t, [c_void_p, c_int]),
    "tq1_linear_chain_f16": (c_int, [c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "tq1_chain_plan_create": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t,
                                      c_void_p, POINTER(c_void_p)]),
    "tq1_chain_plan_run": (c_int, [c_void_p, c_void_p]),
    "tq1_chain_plan_destroy": (None, [c_void_p]),
    "tq1_embedding_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int,
                                  c_void_p]),
}

class Shard(ctypes.Structure):
    """Mirror of ``tq1_shard`` in include/ternel_b200.h."""
    _fields_ = [
        ("rank", c_int), ("world", c_int), ("n_offset", c_int), ("n_total", c_int),
        ("peer_y", c_void_p * 8), ("peer_flags", c_void_p * 8),
        ("epoch_base", c_void_p), ("publish_epoch", ctypes.c_uint32), ("wait_flags", c_void_p),
        ("wait_epoch", ctypes.c_uint32), ("wait_tiles", c_int),
    ]


class ChainLink(ctypes.Structure):
    """Mirror of ``tq1_chain_link`` in include/ternel_b200.h."""
    _fields_ = [
        ("blocks", c_void_p), ("N", c_int), ("K", c_int), ("x", c_void_p), ("source", c_int),
        ("source_offset", c_int), ("y", c_void_p), ("y_is_f32", c_int), ("swiglu", c_int),
        ("out_scale", ctypes.c_float), ("layout", c_int), ("partial", c_int),
    ]


class ChainPeers(ctypes.Structure):
    """Mirror of ``tq1_chain_peers`` in include/ternel_b200.h."""
    _fields_ = [("rank", c_int), ("world", c_int), ("handoff", c_void_p * 8)]


_lib: ctypes.CDLL | None = None

# TERNEL_B200_LIBRARY names another build of the same C ABI to load instead (the bounds-checking build,
# _lib/libternel_b200_checked.so, is the intended use). It is read once, at the first call.
LIBRARY_ENV = "TERNEL_B200_LIBRARY"


class NativeLibraryMissing(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded library; raises loudly if it has not been built."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get(LIBRARY_ENV) or LIB_PATH)
        if not path.exists():
            raise NativeLibraryMissing(
                f"{path} is missing: build it with `python -m ternel_b200.build` "
                "(there is no CPU or PyTorch fallback for the packed ternary kernels)"
            )
        handle = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if hasattr(handle, "tq1_debug_bounds"):         # exported by the bounds-checking build only
            handle.tq1_debug_bounds.restype = c_int
            handle.tq1_debug_bounds.argtypes = [POINTER(ctypes.c_uint64)]
        _lib = handle
    return _lib


def bounds_record() -> "tuple[int, int, int, int] | None":
    """(violations, code of the first, its index, its limit) since the last call, or None when the loaded
    library is not the bounds-checking build. Reading clears the record."""
    handle = lib()
    if not hasattr(handle, "tq1_debug_bounds"):
        return None
    record = (ctypes.c_uint64 * 4)()
    if handle.tq1_debug_bounds(record) != TQ1_OK:
        raise RuntimeError("tq1_debug_bounds: the record could not be read")
    return tuple(int(v) for v in record)


def last_error() -> str:
    return (lib().tq1_last_error() or b"").decode("utf-8", "replace")
