"""B200-native packed ternary (TQ1_G128) linear and embedding path.

Host side in Python over a C-ABI CUDA library (``_lib/libternel_b200.so``,
declared in ``include/ternel_b200.h``); see ``ternel_b200.build`` to compile it.
"""

from .format import (BLOCK_BYTES, BLOCK_SIZE, FormatError, decode_tq1_blocks, encode_tq1_blocks,
                     validate_blocks)
from .layout import (PackedTensorLayout, pack_blocks, select_tile, unpack_blocks,
                     validate_packed_codes)

__all__ = [
    "BLOCK_BYTES", "BLOCK_SIZE", "FormatError", "decode_tq1_blocks", "encode_tq1_blocks",
    "validate_blocks", "PackedTensorLayout", "pack_blocks", "select_tile", "unpack_blocks",
    "validate_packed_codes",
]


def __getattr__(name):
    # torch-dependent names are imported lazily so the codec works without importing torch
    if name in ("PackedLinear", "PackedEmbedding", "packed_matmul"):
        from . import modules
        return getattr(modules, name)
    if name in ("replace_with_packed", "expect_counts", "blocks_from_ternary"):
        from . import packed_model
        return getattr(packed_model, name)
    if name in ("tq1_matmul", "tq1_gemm", "tq1_get_rows", "validate_device_blocks", "tq1_swiglu",
                "interleave_gate_up", "check_status"):
        from . import ops
        return getattr(ops, name)
    if name in ("ChainPlan", "Link", "linear_chain", "blocks_to_panels", "panels_to_blocks", "chain_workspace_bytes"):
        from . import chain
        return getattr(chain, name)
    raise AttributeError(name)
