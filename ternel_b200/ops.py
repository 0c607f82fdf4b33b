"""``torch.library`` custom ops over the C ABI (CUDA only, no fallback).

``ternel::tq1_linear``, ``ternel::tq1_embedding`` and ``ternel::tq1_validate``
take the packed weight as canonical blocks ``uint8[N, K/128, 28]`` resident on
the GPU. PyTorch is only used for device memory and the current stream; the
work happens in ``libternel_b200.so``. The ops are registered for the CUDA
dispatch key alone, so a CPU tensor is refused by the dispatcher instead of
being served by some other path.

The Python wrappers below (`tq1_matmul`, `tq1_gemm`, `tq1_get_rows`) keep the
names and the pre-launch checks of the reference's kernel wrappers
(src/ternel_mlx/kernels.py:1191-1284,1360-1398).
"""

from __future__ import annotations

import ctypes

import torch

from . import _native
from .format import BLOCK_BYTES, BLOCK_SIZE, FormatError, check

ACTIVATION_DTYPES = (torch.float16,)
OUTPUT_DTYPES = (torch.float16, torch.float32)

_workspaces: dict[int, torch.Tensor] = {}


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """A per-device scratch buffer, grown on demand and reused across calls.

    Calls on one device share it, which is safe because they are ordered on the
    current stream; callers that use several streams per device must pass their
    own workspace through the C ABI instead.
    """
    if nbytes == 0:
        return None
    index = device.index if device.index is not None else torch.cuda.current_device()
    buf = _workspaces.get(index)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)   # slots start at zero
        _workspaces[index] = buf
    return buf


def check_status(device=None) -> None:
    """Read the status word of the shared per-device workspace (synchronises the device).

    Zero: every bounded wait inside the kernels was met. 7: results are good but the sequence tags are about
    to wrap, so the workspace is zeroed here. Anything else raises: a wait ran out (the results of the calls
    since the last check are not to be trusted) and the workspace is zeroed so that later calls start clean.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    buf = _workspaces.get(index)
    if buf is None:
        return
    torch.cuda.synchronize(device)
    status = int(buf[:4].view(torch.int32)[0].item())
    if status == 0:
        return
    buf.zero_()
    if status != 7:
        raise RuntimeError(f"a bounded wait inside a packed ternary kernel ran out (status {status}); "
                           "the workspace has been reset")


def _check_blocks(blocks: torch.Tensor) -> tuple[int, int]:
    if blocks.dtype != torch.uint8:
        raise FormatError(f"canonical blocks must be uint8, got {blocks.dtype}")
    if blocks.dim() != 3 or blocks.shape[2] != BLOCK_BYTES:
        raise FormatError(f"blocks must have shape (rows, groups, 28), got {tuple(blocks.shape)}")
    if blocks.shape[0] <= 0 or blocks.shape[1] <= 0:
        raise FormatError("packed tensor has no rows or no groups")
    if not blocks.is_contiguous():
        raise FormatError("blocks must be contiguous")
    return blocks.shape[0], blocks.shape[1]


@torch.library.custom_op("ternel::tq1_linear", mutates_args=(), device_types="cuda")
def _tq1_linear_op(blocks: torch.Tensor, x: torch.Tensor, out_f32: bool) -> torch.Tensor:
    rows, groups = blocks.shape[0], blocks.shape[1]
    batch, columns = x.shape
    out = torch.empty((batch, rows), dtype=torch.float32 if out_f32 else torch.float16, device=x.device)
    lib = _native.lib()
    need = lib.tq1_linear_workspace_bytes(batch, rows, columns)
    ws = _workspace(x.device, need)
    with torch.cuda.device(x.device):
        check(lib.tq1_linear_f16(blocks.data_ptr(), x.data_ptr(), out.data_ptr(), int(out_f32),
                                 batch, rows, columns,
                                 ws.data_ptr() if ws is not None else None,
                                 ws.numel() if ws is not None else 0,
                                 _stream_ptr(x.device)))
    return out


@_tq1_linear_op.register_fake
def _(blocks, x, out_f32):
    return x.new_empty((x.shape[0], blocks.shape[0]), dtype=torch.float32 if out_f32 else torch.float16)


@torch.library.custom_op("ternel::tq1_linear_swiglu", mutates_args=(), device_types="cuda")
def _tq1_linear_swiglu_op(blocks: torch.Tensor, x: torch.Tensor, out_f32: bool) -> torch.Tensor:
    rows = blocks.shape[0]
    batch, columns = x.shape
    out = torch.empty((batch, rows // 2), dtype=torch.float32 if out_f32 else torch.float16, device=x.device)
    lib = _native.lib()
    need = lib.tq1_linear_workspace_bytes(batch, rows, columns)
    ws = _workspace(x.device, need)
    with torch.cuda.device(x.device):
        check(lib.tq1_linear_swiglu_f16(blocks.data_ptr(), x.data_ptr(), out.data_ptr(), int(out_f32),
                                        batch, rows // 2, columns,
                                        ws.data_ptr() if ws is not None else None,
                                        ws.numel() if ws is not None else 0, _stream_ptr(x.device)))
    return out


@_tq1_linear_swiglu_op.register_fake
def _(blocks, x, out_f32):
    return x.new_empty((x.shape[0], blocks.shape[0] // 2), dtype=torch.float32 if out_f32 else torch.float16)


@torch.library.custom_op("ternel::tq1_embedding", mutates_args=(), device_types="cuda")
def _tq1_embedding_op(blocks: torch.Tensor, ids: torch.Tensor, out_f32: bool) -> torch.Tensor:
    rows, groups = blocks.shape[0], blocks.shape[1]
    columns = groups * BLOCK_SIZE
    out = torch.empty((ids.numel(), columns), dtype=torch.float32 if out_f32 else torch.float16,
                      device=blocks.device)
    with torch.cuda.device(blocks.device):
        check(_native.lib().tq1_embedding_f16(blocks.data_ptr(), ids.data_ptr(), out.data_ptr(),
                                              int(out_f32), ids.numel(), rows, columns,
                                              _stream_ptr(blocks.device)))
    return out


@_tq1_embedding_op.register_fake
def _(blocks, ids, out_f32):
    return blocks.new_empty((ids.numel(), blocks.shape[1] * BLOCK_SIZE),
                            dtype=torch.float32 if out_f32 else torch.float16)


@torch.library.custom_op("ternel::tq1_validate", mutates_args=(), device_types="cuda")
def _tq1_validate_op(blocks: torch.Tensor) -> torch.Tensor:
    counts = torch.empty(2, dtype=torch.int64, device=blocks.device)
    groups = blocks.numel() // BLOCK_BYTES
    with torch.cuda.device(blocks.device):
        check(_native.lib().tq1_validate_blocks_device(blocks.data_ptr(), groups, counts.data_ptr(),
                                                       _stream_ptr(blocks.device)))
    return counts


@_tq1_validate_op.register_fake
def _(blocks):
    return blocks.new_empty(2, dtype=torch.int64)


def _require_cuda(tensor: torch.Tensor, name: str) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(
            f"{name} is on {tensor.device}: the packed ternary kernels run on CUDA only "
            "(there is no CPU fallback)")


def validate_device_blocks(blocks: torch.Tensor) -> None:
    """Load-time scan on the GPU; raises FormatError with both counts (fail closed)."""
    _check_blocks(blocks)
    _require_cuda(blocks, "blocks")
    bad_full, bad_tail = (int(v) for v in _tq1_validate_op(blocks).tolist())
    if bad_full or bad_tail:
        raise FormatError(f"invalid base-3 bytes: regular={bad_full}, tail={bad_tail}")


def _check_activations(x: torch.Tensor, groups_per_row: int) -> int:
    if x.dtype not in ACTIVATION_DTYPES:
        raise FormatError(f"activations must be one of {ACTIVATION_DTYPES}, got {x.dtype}")
    if x.dim() != 2:
        raise FormatError(f"activations must be 2-D (batch, columns), got shape {tuple(x.shape)}")
    columns = groups_per_row * BLOCK_SIZE
    if x.shape[1] != columns:
        raise FormatError(f"activations have {x.shape[1]} columns, expected {columns}")
    if x.shape[0] <= 0:
        raise FormatError("activations have an empty batch dimension")
    return x.shape[0]


def tq1_matmul(blocks: torch.Tensor, x: torch.Tensor, *, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ W.T`` for packed ``W``: ``x`` is ``(batch, K)`` FP16, result ``(batch, N)``.

    The output dtype defaults to ``x``'s (one narrowing at the store after FP32
    accumulation, as in the reference); ``torch.float32`` keeps the accumulator.
    The kernel (streaming GEMV, small-batch split-K, or tiled GEMM) is chosen
    inside the library from the batch size.
    """
    _, groups = _check_blocks(blocks)
    _check_activations(x, groups)
    out_dtype = out_dtype or x.dtype
    if out_dtype not in OUTPUT_DTYPES:
        raise FormatError(f"output dtype must be one of {OUTPUT_DTYPES}, got {out_dtype}")
    _require_cuda(blocks, "blocks")
    _require_cuda(x, "activations")
    if blocks.device != x.device:
        raise FormatError(f"blocks on {blocks.device} but activations on {x.device}")
    return _tq1_linear_op(blocks, x.contiguous(), out_dtype == torch.float32)


def tq1_swiglu(blocks: torch.Tensor, x: torch.Tensor, *, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` in one call, for ``blocks`` holding the gate and up rows interleaved
    (row ``2i`` = gate row ``i``, row ``2i + 1`` = up row ``i``; see ``interleave_gate_up``). Dot products and
    the activation are FP32, with one narrowing at the store. Result ``(batch, rows / 2)``."""
    rows, groups = _check_blocks(blocks)
    if rows % 2:
        raise FormatError(f"{rows} rows cannot be (gate, up) pairs")
    _check_activations(x, groups)
    out_dtype = out_dtype or x.dtype
    if out_dtype not in OUTPUT_DTYPES:
        raise FormatError(f"output dtype must be one of {OUTPUT_DTYPES}, got {out_dtype}")
    _require_cuda(blocks, "blocks")
    _require_cuda(x, "activations")
    if blocks.device != x.device:
        raise FormatError(f"blocks on {blocks.device} but activations on {x.device}")
    return _tq1_linear_swiglu_op(blocks, x.contiguous(), out_dtype == torch.float32)


def interleave_gate_up(gate_blocks: torch.Tensor, up_blocks: torch.Tensor) -> torch.Tensor:
    """Canonical blocks with gate row ``i`` at row ``2i`` and up row ``i`` at row ``2i + 1`` (a byte copy)."""
    _check_blocks(gate_blocks)
    _check_blocks(up_blocks)
    if gate_blocks.shape != up_blocks.shape:
        raise FormatError(f"gate {tuple(gate_blocks.shape)} and up {tuple(up_blocks.shape)} differ in shape")
    return torch.stack((gate_blocks, up_blocks), dim=1).reshape(2 * gate_blocks.shape[0], *gate_blocks.shape[1:]).contiguous()


# The reference exposes the prefill kernel under its own name; here both names
# reach the same entry point, which picks the kernel from the batch size.
tq1_gemm = tq1_matmul


def tq1_get_rows(blocks: torch.Tensor, indices: torch.Tensor, *, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Decode the rows named by 1-D ``indices``; an id outside ``[0, rows)`` gives a zero row."""
    _check_blocks(blocks)
    if dtype not in OUTPUT_DTYPES:
        raise FormatError(f"output dtype must be one of {OUTPUT_DTYPES}, got {dtype}")
    if indices.dtype.is_floating_point or indices.dtype == torch.bool or indices.dtype.is_complex:
        raise FormatError(f"indices must be an integer tensor, got {indices.dtype}")
    if indices.dim() != 1:
        raise FormatError(f"indices must be 1-D, got shape {tuple(indices.shape)}")
    if indices.numel() <= 0:
        raise FormatError("indices are empty")
    _require_cuda(blocks, "blocks")
    ids = indices.to(device=blocks.device, dtype=torch.int64).contiguous()
    return _tq1_embedding_op(blocks, ids, dtype == torch.float32)
