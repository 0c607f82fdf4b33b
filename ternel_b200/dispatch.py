"""Which kernel and tiling a linear call takes, and the recorded sweep the rule was chosen from.

The reference chooses its kernel configuration per batch size from committed sweeps and replays
them in its tests (``select_lut23`` / ``select_gemm``, src/ternel_mlx/modules.py:331-422;
tests/test_mlx_modules.py:553-1084). Here the choice lives in the C library (``tq1_linear_plan``)
and the sweep it was chosen from is ``dispatch_sweep_b200.json`` beside this file:

    python -m ternel_b200.dispatch --out ternel_b200/dispatch_sweep_b200.json    # on a B200

records, for every batch size and shape of the sweep, the time of every token tile the
tensor-core kernel can run with and, for batches up to ``LOOPED_MAX``, the time of the same call
as passes of the batch-1 kernel in one launch; ``tests/test_dispatch_replay.py`` checks that the
rule's choice is within a few percent of the best recorded one everywhere.
"""

from __future__ import annotations

import argparse
import ctypes
import json
from dataclasses import dataclass
from pathlib import Path

from . import _native
from .format import check

SWEEP_PATH = Path(__file__).resolve().parent / "dispatch_sweep_b200.json"
KERNELS = {0: "rows", 1: "stream_gemv", 2: "tensor_core"}
TOKEN_TILES = (16, 32, 64, 128, 256)
LOOPED_MAX = 4          # largest batch also timed as passes of the batch-1 kernel
SWEEP_BATCHES = (2, 3, 4, 8, 16, 17, 24, 32, 33, 48, 64, 65, 96, 128, 192, 256, 512, 1023, 1024, 2048)
SWEEP_SHAPES = ((5120, 5120), (1024, 5120), (17408, 5120), (5120, 17408))


@dataclass(frozen=True)
class LinearPlan:
    kernel: str          # "rows", "stream_gemv" or "tensor_core"
    token_tile: int      # activation rows per tile (tensor-core kernel), else 0
    ctas: int
    parts: int           # equal K parts per tile, 0 = stream-K ranges


def plan(batch: int, rows: int, columns: int, *, aligned: bool = True) -> LinearPlan:
    """The library's choice for ``x[batch, columns] @ W[rows, columns].T`` (launches nothing)."""
    kernel, tile, ctas, parts = (ctypes.c_int() for _ in range(4))
    check(_native.lib().tq1_linear_plan(batch, rows, columns, int(aligned), ctypes.byref(kernel), ctypes.byref(tile),
                                        ctypes.byref(ctas), ctypes.byref(parts)))
    return LinearPlan(KERNELS[kernel.value], tile.value, ctas.value, parts.value)


def looped_tokens() -> int:
    """Largest batch the library runs as passes of the batch-1 kernel (found by probing the plan)."""
    tokens = 1
    while tokens < 8 and plan(tokens + 1, 5120, 5120).kernel == "stream_gemv":
        tokens += 1
    return tokens


def chosen_over_best(case: dict) -> "tuple[float, LinearPlan]":
    """Recorded time of the library's choice for a sweep case over the best recorded option of that case."""
    options = {int(k): v for k, v in case["us_by_token_tile"].items()}
    best = min(options.values())
    if "us_looped" in case:
        best = min(best, case["us_looped"])
    chosen = plan(case["batch"], case["rows"], case["columns"])
    took = case["us_looped"] if chosen.kernel == "stream_gemv" else options[chosen.token_tile]
    return took / best, chosen


def load_sweep(path: Path = SWEEP_PATH) -> dict:
    return json.loads(Path(path).read_text())


def record_sweep(batches=SWEEP_BATCHES, shapes=SWEEP_SHAPES, tiles=TOKEN_TILES, ring: int = 6, replays: int = 3) -> dict:
    """Time every (batch, shape, token tile) on the current GPU: CUDA-graph replays over a ring of
    distinct weight buffers, CUDA events. Returns the JSON-ready record."""
    import torch
    from .stack import random_blocks_device

    default_loop = looped_tokens()
    lib = _native.lib()
    lib.tq1_debug_set_loop_tokens.restype = ctypes.c_int
    lib.tq1_debug_set_loop_tokens.argtypes = [ctypes.c_int]
    device = torch.device("cuda")
    gen = torch.Generator(device=device)
    gen.manual_seed(7)
    cases = []

    def time_call(weights, x, y, batch, rows, columns):
        need = lib.tq1_linear_workspace_bytes(batch, rows, columns)
        ws = torch.zeros(need, dtype=torch.uint8, device=device)

        def run():
            stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            for w in weights:
                check(lib.tq1_linear_f16(w.data_ptr(), x.data_ptr(), y.data_ptr(), 0, batch, rows, columns,
                                         ws.data_ptr(), need, stream))

        torch.cuda.synchronize()
        side = torch.cuda.Stream(device=device)
        with torch.cuda.stream(side):
            run()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run()
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        del graph
        return round(start.elapsed_time(stop) * 1e3 / (replays * len(weights)), 3)

    try:
        for rows, columns in shapes:
            weights = [random_blocks_device(rows, columns, gen, device) for _ in range(ring)]
            for batch in batches:
                x = torch.randn((batch, columns), generator=gen, device=device).to(torch.float16)
                y = torch.empty((batch, rows), dtype=torch.float16, device=device)
                times = {}
                check(lib.tq1_debug_set_loop_tokens(0))        # the tensor-core kernel, tile by tile
                for tile in tiles:
                    if tile > 16 and tile >= 4 * batch:       # a tile mostly of padding: not a candidate
                        continue
                    check(lib.tq1_debug_force_token_tile(tile))
                    times[str(tile)] = time_call(weights, x, y, batch, rows, columns)
                case = {"batch": batch, "rows": rows, "columns": columns, "us_by_token_tile": times}
                if batch <= LOOPED_MAX:                        # the same call as passes of the batch-1 kernel
                    check(lib.tq1_debug_force_token_tile(0))
                    check(lib.tq1_debug_set_loop_tokens(batch))
                    case["us_looped"] = time_call(weights, x, y, batch, rows, columns)
                cases.append(case)
            del weights
    finally:
        check(lib.tq1_debug_force_token_tile(0))
        check(lib.tq1_debug_set_loop_tokens(default_loop))
    return {"device": torch.cuda.get_device_name(device), "ring_buffers": ring,
            "unit": "microseconds per call, CUDA-graph replays, distinct weight buffers", "cases": cases}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--out", type=Path, default=SWEEP_PATH)
    args = parser.parse_args()
    record = record_sweep()
    args.out.write_text(json.dumps(record, indent=1) + "\n")
    worst = max(chosen_over_best(case)[0] for case in record["cases"])
    print(f"wrote {args.out} ({len(record['cases'])} cases); the rule's worst case is {worst:.3f}x the best recorded option")


if __name__ == "__main__":
    main()
