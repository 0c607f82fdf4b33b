"""Benchmark of the packed ternary (TQ1_G128) decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step at batch ``--batch`` over a synthetic 27B-class
dense decoder: ``--layers`` (64) layers x 7 projections (q/o 5120x5120, k/v
1024x5120, gate/up 17408x5120, down 5120x17408; 4.62 GB of packed weights, far
larger than the 126 MB L2, so every step streams from HBM) plus one packed
embedding row gather per sequence. With N > 1 every projection is
output-row-sharded over the ranks and the FP16 output shards are all-gathered
after each projection (strong scaling: the total work per step is fixed).

The metric is effective HBM bandwidth of the packed GEMV path: algorithmic
bytes (28 B per 128 weights + FP16 activations in + FP16 results out) moved by
all ranks per second. ``tokens_per_s`` (= batch / step time) is printed beside it.

Rank 0 prints exactly one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "tq1_gemv_effective_hbm_gbps"
UNIT = "GB/s"


NCU_TRAFFIC_RATIO = 72.93 / 72.42     # measured DRAM bytes / algorithmic bytes, batch-1 GEMV, four shapes


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--impl", choices=("ours", "reference"), default="ours")
    p.add_argument("--layers", type=int, default=64)
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--no-graph", action="store_true", help="launch every kernel from the host each step")
    p.add_argument("--unfused", action="store_true",
                   help="seven launches per layer (q,k,v,o,gate,up,down) instead of four (qkv,o,gate_up,down)")
    p.add_argument("--exchange", choices=("p2p", "nccl"), default="p2p",
                   help="how row shards are gathered when --gpus > 1: pushed by the kernels, or NCCL all-gather")
    p.add_argument("--skip-cpu-baseline", action="store_true")
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--skip-batched", action="store_true", help="skip the small-batch and prefill side measurements")
    p.add_argument("--only-batched", default="",
                   help="run only the batched side measurement on these cases, e.g. '2:17408x5120,2048:5120x17408' "
                        "(M:NxK), print its JSON and exit; with --ring to choose the number of distinct weight buffers")
    p.add_argument("--ring", type=int, default=14, help="distinct weight buffers per shape in the batched measurement")
    p.add_argument("--only-gather", type=int, default=0, metavar="TOKENS",
                   help="time only the packed-embedding gather of this many token ids (151936 x 5120 table), "
                        "print its JSON and exit")
    return p.parse_args()


def workload_config(args) -> dict:
    return {
        "workload": "decode_step_27b_class_layers",
        "layers": args.layers,
        "batch": args.batch,
        "shapes_NxK": ["5120x5120 (q,o)", "1024x5120 (k,v)", "17408x5120 (gate,up)", "5120x17408 (down)"],
        "embedding": "151936x5120 packed, one row per sequence",
        "launches_per_layer": "7 (q,k,v,o,gate,up,down)" if args.unfused else
                              "4 (q|k|v and gate|up stored row-concatenated: 7168x5120, 5120x5120, 34816x5120, 5120x17408)",
        "packed_weight_bytes": None,   # filled in
        "parallelism": (f"row-sharded x{args.gpus}, shards exchanged by "
                        + ("kernel epilogue pushes over NVLink + flags" if args.exchange == "p2p" else "NCCL all-gather")
                        if args.gpus > 1 else "single GPU"),
        "l2_policy": "inputs larger than L2 (each step streams every layer's distinct weights)",
    }


# ----------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores
# ----------------------------------------------------------------------------

def time_cpu_layer(batch: int, budget_s: float, min_reps: int = 1):
    """Time the C restatement of the reference's decode-and-dot on ONE layer's 7 projections."""
    import numpy as np
    from oracle import c_oracle, tq1_oracle as o
    from ternel_b200.stack import LayerShape

    shape = LayerShape()
    rng = np.random.default_rng(0)
    mats = []
    for _, n, k in shape.projections():
        groups = n * k // 128
        blocks = rng.integers(0, 243, size=(groups, 28), dtype=np.uint8)   # legal bytes; timing only
        blocks[:, 27] %= 27
        blocks[:, 1] = (blocks[:, 1] & 0x03) | 0x20                        # modest finite scales
        x = rng.standard_normal((batch, k)).astype(np.float16).astype(np.float32)
        mats.append((blocks, x, n, k))
    # prove the port right on a small case before timing it
    small, xs = o.synth_matrix(256, 1280, seed=3)
    want = o.float64_matmul(small, xs[None].astype(np.float32), rows=256, columns=1280)
    got = c_oracle.matmul_f32(small, xs[None].astype(np.float32), rows=256, columns=1280)
    assert o.normalised_error(got, want) < 1e-5
    threads = c_oracle.threads()
    times = []
    start = time.perf_counter()
    while len(times) < min_reps or (time.perf_counter() - start < budget_s and len(times) < 50):
        t0 = time.perf_counter()
        for blocks, x, n, k in mats:
            c_oracle.matmul_f32(blocks, x, rows=n, columns=k, threads=threads)
        times.append(time.perf_counter() - t0)
    times.sort()
    median = times[len(times) // 2]
    alg_bytes = sum(n * k // 128 * 28 + 2 * batch * (n + k) for _, _, n, k in mats)
    return alg_bytes / median / 1e9, threads, len(times), median


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # each step = one layer (1/64 of the decode step) on all host cores
    import numpy as np
    gbps_samples = []
    value = threads = None
    for _ in range(max(1, args.warmup // 3)):
        time_cpu_layer(args.batch, 0.0)
    t_all = []
    for _ in range(args.steps):
        v, threads, _, sec = time_cpu_layer(args.batch, 0.0)
        gbps_samples.append(v)
        t_all.append(sec)
    value = float(np.median(gbps_samples))
    ms = float(np.median(t_all)) * 1e3
    cfg = workload_config(args)
    cfg["packed_weight_bytes"] = 72253440 * args.layers
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "one of the 64 layers (7 projections, 72.3 MB packed) per step, "
                                   "C restatement of the reference's NumPy decode-and-dot on all host cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": args.batch / (ms * args.layers / 1e3),
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu_index), "-lms", "20"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().strip().splitlines() if r.strip()]
        os.unlink(self.file.name)
        sm, mx, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); power.append(float(r[3]))
            except ValueError:
                continue
            for name, flag in zip(names, r[5:9]):
                if flag.strip().lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def run_gpu_arm(args) -> None:
    import torch
    import torch.distributed as dist
    from ternel_b200.stack import LayerShape, LayerStack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stack = LayerStack(layers=args.layers, batch=args.batch, vocab=151936, rank=rank, world=world,
                       device=device, seed=0, fused=not args.unfused, exchange=args.exchange)
    # correctness before timing: one projection of this rank against the C oracle
    # (every rank runs the step: sharded steps exchange data and must stay in lockstep)
    stack.step()
    barrier()
    if rank == 0:
        from oracle import c_oracle, tq1_oracle as o
        name, n, k = stack.projections[-1]     # the last writer of its output buffer
        blocks = stack.weights[-1][-1].cpu().numpy()
        x = stack.inputs[k].float().cpu().numpy()
        want = c_oracle.matmul_f32(blocks, x, rows=n // world, columns=k)
        if world > 1 and stack.exchange == "p2p":
            got = stack.outputs[n][:, : n // world].float().cpu().numpy()
        else:
            got = (stack.outputs[n][0] if world > 1 else stack.outputs[n]).float().cpu().numpy().reshape(args.batch, -1)
        err = o.normalised_error(got, want)
        assert err < 2e-3, f"parity check failed before timing: {err}"

    # the NCCL baseline exchange is launched from the host every step (its capture did not complete here)
    use_graph = not args.no_graph and not (world > 1 and args.exchange == "nccl")
    graph = None
    if use_graph:
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            stack.step()            # warm every kernel/attribute before capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            stack.step()

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            stack.step()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()             # nvidia-smi needs a moment to start: sample from the warm-up on
    for _ in range(max(args.warmup, 3)):
        one_step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        one_step()
    stop.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = start.elapsed_time(stop)
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    alg_bytes_rank = stack.algorithmic_bytes_per_step
    alg_bytes_all = alg_bytes_rank * world
    value = alg_bytes_all / (ms_per_step / 1e3) / 1e9

    per_shape = measure_shapes(stack, device) if world == 1 else None
    batched = measure_batched(device) if world == 1 and not args.skip_batched else None
    if batched is not None and args.batch == 1:
        batched["decode_step_batch8"] = measure_step_batch8(args, stack, device)
        batched["gather"] = [measure_gather(tokens, table=stack.table) for tokens in (512, 8192)]

    # end-to-end through the public operator API with host buffers
    e2e = None
    if not args.skip_e2e:
        e2e = measure_e2e(args, stack, device, world, barrier, one_step)

    checksum = stack.checksum()
    status = int(stack.workspace[:4].view(torch.int32)[0].item())
    if status != 0:
        raise SystemExit(f"rank {rank}: a bounded device wait ran out (status word {status}); the run is void")
    if rank == 0:
        peaks = {}
        peaks_path = ROOT / "MEASURED_PEAKS.json"
        if peaks_path.exists():
            peaks = json.loads(peaks_path.read_text())
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
        per_gpu = alg_bytes_rank / (ms_per_step / 1e3) / 1e9
        cfg = workload_config(args)
        cfg["packed_weight_bytes"] = stack.packed_bytes_per_step * world
        cfg["cuda_graph"] = use_graph
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "tokens_per_s": args.batch / (ms_per_step / 1e3),
            "gpu_launches": stack.launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {
                "bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                "frac_of_nominal_8000": per_gpu / 8000.0, "peak_source": peak_kind,
                "kernel": "packed GEMV (all projections of the step)",
                "algorithmic_bytes_per_launch_avg": alg_bytes_rank / stack.launches_per_step,
                "avg_launch_us": ms_per_step * 1e3 / stack.launches_per_step,
                # DRAM bytes per launch: the ncu capture of one launch of each of the four shapes
                # (the committed ncu summary of the batch-1 kernel) read 72.93 MB against 72.42 MB of
                # algorithmic bytes; traffic grows with the units processed, so the ratio carries over.
                # Only the fused batch-1 single-GPU step was captured.
                "traffic": (NCU_TRAFFIC_RATIO * alg_bytes_rank / stack.launches_per_step
                            if args.batch == 1 and world == 1 and not args.unfused else None),
                "traffic_source": "ncu dram__bytes_read+write of a 2-layer capture, scaled by bytes processed",
            },
            "checksum": checksum,
        }
        if e2e is not None:
            line["e2e"] = e2e
        if per_shape is not None:
            line["per_shape"] = per_shape
        if batched is not None:
            line["batched"] = batched
        if world == 1 and not args.skip_cpu_baseline:
            v, threads, reps, sec = time_cpu_layer(args.batch, budget_s=12.0, min_reps=3)
            line["cpu_baseline"] = {
                "value": v, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"one of the {args.layers} layers (7 projections, 72.3 MB packed), median of {reps} "
                          f"passes of the C restatement of the reference's NumPy decode-and-dot "
                          f"({sec * 1e3:.1f} ms per layer)",
            }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_shapes(stack, device, replays: int = 5):
    """Per projection shape, one CUDA graph of back-to-back launches: the stream regime (the same
    projection of every layer, distinct weight buffers, far more than L2 in total: the HBM number) and the
    warm regime (one buffer repeatedly: L2-resident weights). The chained regime is the step itself."""
    import ctypes
    import torch
    from ternel_b200.format import check

    lib = stack.lib
    out = {}
    seen = set()
    for j, (name, n, k) in enumerate(stack.projections):
        if (n, k) in seen:
            continue
        seen.add((n, k))

        def timed(same_buffer: bool) -> float:
            """us per launch of one CUDA graph holding len(stack.weights) launches of this shape."""
            def run():
                stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
                for layer in stack.weights:
                    blocks = stack.weights[0][j] if same_buffer else layer[j]
                    check(lib.tq1_linear_f16(blocks.data_ptr(), stack.inputs[k].data_ptr(),
                                             stack.outputs[n].data_ptr(), 0, stack.batch, n, k,
                                             stack.workspace.data_ptr(), stack.workspace_bytes, stream))

            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
            for _ in range(2):
                graph.replay()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(replays):
                graph.replay()
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop) * 1e3 / (replays * len(stack.weights))

        us = timed(False)           # stream regime: distinct buffers, HBM
        warm = timed(True)          # warm regime: one buffer over and over, L2
        alg = n * k // 128 * 28 + 2 * stack.batch * (n + k)
        out[f"{n}x{k}"] = {"us_per_launch": us, "gbps": alg / us / 1e3, "ring_buffers": len(stack.weights),
                           "warm_l2_us_per_launch": warm, "warm_l2_gbps": alg / warm / 1e3}
    return out


def measure_batched(device, replays: int = 3, cases=None, ring_size: int = 14):
    """Side measurements of the batched kernels: small batch (M = 2..16, HBM-bound, GB/s of packed
    weights) and prefill (M = 512, 2048, tensor-bound, TFLOP/s), each over a ring of distinct weights."""
    import ctypes
    import torch
    from ternel_b200 import _native
    from ternel_b200.format import check
    from ternel_b200.stack import random_blocks_device

    lib = _native.lib()
    gen = torch.Generator(device=device)
    gen.manual_seed(123)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak_tf = float(json.loads(peaks_path.read_text()).get("bf16_tflops", 1590.0)) if peaks_path.exists() else 1590.0
    out = {"small_batch": {}, "prefill": {}, "tensor_peak_tflops": peak_tf}
    if cases is None:
        cases = [(m, n, k) for n, k in ((17408, 5120), (5120, 17408)) for m in (2, 4, 8, 16, 512, 2048)]
    for n, k in dict.fromkeys((n, k) for _, n, k in cases):
        ring = [random_blocks_device(n, k, gen, device) for _ in range(ring_size)]   # 14 x 19.5 MB > 2 x L2
        for m in [m for m, n2, k2 in cases if (n2, k2) == (n, k)]:
            x = torch.randn((m, k), generator=gen, device=device).to(torch.float16)
            y = torch.empty((m, n), dtype=torch.float16, device=device)
            ws_bytes = lib.tq1_linear_workspace_bytes(m, n, k)
            ws = torch.zeros(max(ws_bytes, 256), dtype=torch.uint8, device=device)

            def run():
                stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
                for w in ring:
                    check(lib.tq1_linear_f16(w.data_ptr(), x.data_ptr(), y.data_ptr(), 0, m, n, k,
                                             ws.data_ptr(), ws_bytes, stream))

            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()        # device time, not the host's launch rate
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
            us = start.elapsed_time(stop) * 1e3 / (replays * len(ring))
            if m <= 16:
                alg = n * k // 128 * 28 + 2 * m * (n + k)
                out["small_batch"][f"M{m}_{n}x{k}"] = {"us": us, "gbps": alg / us / 1e3}
            else:
                tf = 2.0 * m * n * k / us / 1e6
                out["prefill"][f"M{m}_{n}x{k}"] = {"us": us, "tflops": tf, "frac_of_measured_peak": tf / peak_tf}
            del graph, x, y, ws
        del ring
    return out


def measure_gather(tokens: int, vocab: int = 151936, hidden: int = 5120, replays: int = 20, table=None):
    """The packed-embedding gather on its own: `tokens` random ids per call, checked against the oracle on a
    sample, timed with CUDA events. Algorithmic bytes per token: 28*K/128 read + 2*K written."""
    import numpy as np
    import torch
    from oracle import tq1_oracle as o
    from ternel_b200.ops import tq1_get_rows
    from ternel_b200.stack import random_blocks_device

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(5)
    if table is None:
        table = random_blocks_device(vocab, hidden, gen, device)
    vocab, hidden = table.shape[0], table.shape[1] * 128
    ids = torch.randint(0, vocab, (tokens,), generator=gen, device=device)
    out = tq1_get_rows(table, ids)
    torch.cuda.synchronize()
    sample = ids[:8].cpu().numpy()
    sample_rows = table[ids[:8]].cpu().numpy()            # only the sampled rows leave the device
    want = o.get_rows(sample_rows, np.arange(sample.size), rows=sample.size, columns=hidden, dtype=np.float16)
    assert np.array_equal(out[:8].cpu().numpy(), want), "gather parity failed before timing"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)        # larger than L2
    pairs = 8

    def timed_graph(with_gather: bool) -> float:
        """Device time of `pairs` x (L2 flush [+ gather]) captured as one CUDA graph, per pair, in us."""
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            flush.zero_()
            torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for _ in range(pairs):
                flush.zero_()
                if with_gather:
                    tq1_get_rows(table, ids)
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(replays):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e3 / (replays * pairs)

    us = timed_graph(True) - timed_graph(False)      # the flush alone is timed the same way and subtracted
    alg = tokens * (hidden // 128 * 28 + 2 * hidden)
    return {"tokens": tokens, "us": us, "gbps": alg / us / 1e3, "algorithmic_bytes": alg,
            "l2_policy": "256 MiB written between calls (its time measured alone and subtracted), CUDA-graph replays"}


def measure_step_batch8(args, stack, device, replays: int = 10):
    """The same 64-layer step with eight sequences per step (the small-batch kernel), over the same
    resident weights; graph-timed like the headline step."""
    import torch
    from ternel_b200.stack import LayerStack

    stack8 = LayerStack(layers=args.layers, batch=8, vocab=stack.vocab, device=device, seed=0,
                        fused=stack.fused, weights_from=stack)
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        stack8.step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        stack8.step()
    for _ in range(3):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / replays
    status = int(stack8.workspace[:4].view(torch.int32)[0].item())
    if status != 0:
        raise SystemExit(f"batch-8 step: a bounded device wait ran out (status word {status})")
    return {"ms_per_step": ms, "tokens_per_s": 8 / (ms / 1e3),
            "gbps": stack8.algorithmic_bytes_per_step / (ms / 1e3) / 1e9, "checksum": stack8.checksum()}


def measure_e2e(args, stack, device, world, barrier, one_step):
    """Same step through the public API, inputs in pinned host memory every step: the torch custom ops on
    one GPU; on several GPUs the sharded entry (LayerStack's captured step with kernel-side pushes)."""
    import torch
    import torch.distributed as dist
    from ternel_b200.ops import tq1_get_rows, tq1_matmul

    host_x = {k: v.cpu().pin_memory() for k, v in stack.inputs.items()}
    host_ids = stack.ids.cpu().pin_memory()
    last = [(n, torch.empty((args.batch, n), dtype=torch.float16).pin_memory())
            for n in sorted(stack.outputs)]
    h2d = sum(v.numel() * 2 for v in host_x.values()) + host_ids.numel() * 8
    d2h = sum(buf.numel() * 2 for _, buf in last)

    keys = sorted(host_x)

    def forward(ids, *xs):
        """The decode step through the public modules' kernels, device tensors in and out."""
        dev_x = dict(zip(keys, xs))
        tq1_get_rows(stack.table, ids)
        outs = {}
        for layer in stack.weights:
            for (_, n, k), blocks in zip(stack.projections, layer):
                y = tq1_matmul(blocks, dev_x[k])
                if world > 1:
                    full = torch.empty((world, args.batch, n // world), dtype=torch.float16, device=device)
                    dist.all_gather_into_tensor(full, y, group=stack.group)
                    y = full.permute(1, 0, 2).reshape(args.batch, n)
                outs[n] = y
        return tuple(outs[n] for n, _ in last)

    graphed = None
    if world == 1 and not args.no_graph:
        from ternel_b200.graphs import GraphedStep
        graphed = GraphedStep(forward, [stack.ids] + [stack.inputs[k] for k in keys])

    sharded = world > 1 and stack.exchange == "p2p"

    def step():
        if sharded:                     # host -> the stack's static inputs, its captured step, device -> host
            stack.ids.copy_(host_ids, non_blocking=True)
            for k in keys:
                stack.inputs[k].copy_(host_x[k], non_blocking=True)
            one_step()
            for n, buf in last:
                buf.copy_(stack.outputs[n], non_blocking=True)
            torch.cuda.synchronize()
            return
        if graphed is not None:         # host -> static device inputs, one graph replay, device -> host
            outs = graphed(host_ids, *[host_x[k] for k in keys])
        else:
            outs = forward(host_ids.to(device, non_blocking=True),
                           *[host_x[k].to(device, non_blocking=True) for k in keys])
        for (n, buf), y in zip(last, outs):
            buf.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    steps = max(3, min(args.steps, 20))
    for _ in range(3):
        step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    barrier()
    sec = (time.perf_counter() - t0) / steps
    t = torch.tensor([sec], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t.item())
    return {"value": stack.algorithmic_bytes_per_step * world / sec / 1e9, "unit": UNIT,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": sec * 1e3,
            "steps": steps,
            "api": ("ternel_b200.stack.LayerStack.step (tq1_linear_f16_sharded per projection, tq1_embedding_f16), "
                    "captured once as a CUDA graph and replayed" if sharded else
                    "torch.ops.ternel.tq1_linear / tq1_embedding, one call per projection"
                    + (", captured once by ternel_b200.graphs.GraphedStep and replayed" if graphed is not None else ""))}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.only_gather:
        print(json.dumps({"gather": measure_gather(args.only_gather)}))
    elif args.only_batched:
        import torch
        cases = []
        for item in args.only_batched.split(","):
            m, shape = item.split(":")
            n, k = shape.lower().split("x")
            cases.append((int(m), int(n), int(k)))
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        print(json.dumps({"batched": measure_batched(device, cases=cases, ring_size=args.ring)}))
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
