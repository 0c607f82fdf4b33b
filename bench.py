"""Benchmark of the packed ternary (TQ1_G128) decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step at batch ``--batch`` over a synthetic 27B-class
dense decoder: ``--layers`` (64) layers x 7 projections (q/o 5120x5120, k/v
1024x5120, gate/up 17408x5120, down 5120x17408; 4.62 GB of packed weights, far
larger than the 126 MB L2, so every step streams from HBM) plus one packed
embedding row gather per sequence. At batch 1 the whole step is one persistent
launch (a chain of 256 links) in which every projection reads the output of the
one before it, as a decoder's do. With N > 1 every projection is
output-row-sharded over the ranks and every finished output is pushed to all
ranks by the kernel itself (strong scaling: the total work per step is fixed).

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


NCU_TRAFFIC_RATIO = (145.336 + 4.787) / 144.858     # DRAM read + write over algorithmic bytes, one 8-link chain launch


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
    p.add_argument("--exchange", choices=("chain", "nccl"), default="chain",
                   help="batch-1 step as one persistent chain launch (shards pushed by the kernel when --gpus > 1), "
                        "or one launch per projection over fixed inputs with an NCCL all-gather per projection")
    p.add_argument("--independent", action="store_true",
                   help="chain links read fixed synthetic activations instead of each other's outputs")
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
                        + ("the chain kernel: tagged 64-bit words pushed to every rank over NVLink"
                           if args.exchange == "chain" and args.batch == 1 else "NCCL all-gather")
                        if args.gpus > 1 else "single GPU"),
        "step_launch": ("one persistent chain launch, every projection reads the previous one's output"
                        if args.exchange == "chain" and args.batch == 1 and not args.independent else
                        "one persistent chain launch over fixed inputs" if args.exchange == "chain" and args.batch == 1
                        else "one launch per projection over fixed inputs"),
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


def foreign_compute_processes(own_pids=()) -> list:
    """PIDs of other processes with a CUDA context on this box's GPUs (read-only query); a timed unit that
    saw one is marked, as the reference's environment record does (src/bonsai_tq1/environment.py:44-47)."""
    try:
        out = subprocess.run(["nvidia-smi", "--query-compute-apps=pid,used_memory", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=10).stdout
    except (OSError, subprocess.TimeoutExpired):
        return ["nvidia-smi unavailable"]
    mine = {os.getpid(), os.getppid(), *own_pids}
    pids = []
    for row in out.strip().splitlines():
        try:
            pid = int(row.split(",")[0])
        except ValueError:
            continue
        if pid not in mine:
            pids.append(pid)
    return pids


def sample_stats(samples_ms, resamples: int = 20000, seed: int = 0) -> dict:
    """Median, p5/p95 and a bootstrap 95% interval of the median of per-step times (the statistics of the
    reference's reports, src/bonsai_tq1/lut23_reporting.py:65-107)."""
    import numpy as np
    a = np.asarray(samples_ms, dtype=np.float64)
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, a.size, size=(resamples, a.size))
    med = np.median(a[idx], axis=1)
    return {"n": int(a.size), "median_ms": float(np.median(a)), "p5_ms": float(np.percentile(a, 5)),
            "p95_ms": float(np.percentile(a, 95)), "median_ci95_ms": [float(np.percentile(med, 2.5)),
                                                                      float(np.percentile(med, 97.5))]}


def verify_chain(stack, world: int, rank: int) -> dict:
    """Parity of the chained step on EVERY rank, after one step has run: for the links of the first two layers
    and of the last layer, this rank's output rows against the C oracle applied to this rank's weight rows and
    the activations the link actually read -- the FP16 outputs of its source link gathered from all ranks with
    a plain NCCL all-gather. A row that another GPU pushed wrongly, late or torn would change what the next
    link computes here."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import c_oracle, tq1_oracle as o

    links, outs = stack.plan.links, stack.link_outputs
    per_layer = len(stack.projections)
    wanted = sorted(set(range(min(2 * per_layer, len(links)))) | set(range(len(links) - per_layer, len(links))))
    sources = sorted({links[i].source for i in wanted if links[i].x is None})

    def gathered(i):
        y = outs[i]
        if world == 1:
            return y.to(torch.float16) if links[i].partial else y
        if links[i].partial:        # a column shard: what the next link reads is the sum of the ranks' partial sums
            total = y.clone()
            dist.all_reduce(total)
            return total.to(torch.float16)
        full = torch.empty((world, y.numel()), dtype=y.dtype, device=y.device)
        dist.all_gather_into_tensor(full, y.contiguous())
        return full.reshape(-1)

    full_out = {i: gathered(i).float().cpu().numpy() for i in sources}      # every rank takes part in every gather
    worst = 0.0
    for i in wanted:
        link = links[i]
        k = link.columns
        if link.x is not None:
            x = link.x.float().cpu().numpy()
        else:
            x = full_out[link.source][link.source_offset: link.source_offset + k]
        canonical = stack.weights[i // per_layer][i % per_layer]      # the link may stream a permuted copy of these bytes
        want = c_oracle.matmul_f32(canonical.cpu().numpy(), x[None, :].astype(np.float32), rows=link.rows, columns=k)[0]
        if link.swiglu:
            gate, up = want[0::2], want[1::2]
            want = gate / (1.0 + np.exp(-gate)) * up
        want = want * np.float32(link.out_scale)
        got = outs[i].float().cpu().numpy()
        err = o.normalised_error(got[None, :], want[None, :])
        assert np.isfinite(got).all() and np.abs(got).max() > 0, f"rank {rank}: link {i} produced no finite output"
        assert err < 2e-3, f"rank {rank}: link {i} differs from the oracle by {err}"
        worst = max(worst, err)
    ranks_checked = 1
    if world > 1:
        flags = torch.tensor([1.0], device=outs[0].device)
        dist.all_reduce(flags)
        ranks_checked = int(flags.item())
        w = torch.tensor([worst], dtype=torch.float64, device=outs[0].device)
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        worst = float(w.item())
    return {"ranks_checked": ranks_checked, "links_checked": len(wanted), "max_err": worst,
            "bound": 2e-3, "against": "C restatement of the reference's decode-and-dot, inputs = gathered FP16 outputs"}


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

    chain = args.exchange == "chain" and args.batch == 1
    stack = LayerStack(layers=args.layers, batch=args.batch, vocab=151936, rank=rank, world=world,
                       device=device, seed=0, fused=not args.unfused,
                       exchange="chain" if chain else "launches", dependent=not args.independent)
    # correctness before timing (every rank runs the step: sharded steps exchange data and must stay in lockstep)
    stack.step()
    barrier()
    if stack.status() != 0:
        raise SystemExit(f"rank {rank}: a bounded device wait ran out (status word {stack.status()})")
    parity = None
    if chain:
        parity = verify_chain(stack, world, rank)
    elif rank == 0:
        from oracle import c_oracle, tq1_oracle as o
        name, n, k = stack.projections[-1]     # the last writer of its output buffer
        blocks = stack.weights[-1][-1].cpu().numpy()
        x = stack.inputs[k].float().cpu().numpy()
        want = c_oracle.matmul_f32(blocks, x, rows=n // world, columns=k)
        got = (stack.outputs[n][0] if world > 1 else stack.outputs[n]).float().cpu().numpy().reshape(args.batch, -1)
        err = o.normalised_error(got, want)
        assert err < 2e-3, f"parity check failed before timing: {err}"
        parity = {"ranks_checked": 1, "links_checked": 1, "max_err": err, "bound": 2e-3}

    # the NCCL baseline exchange is launched from the host every step
    use_graph = not args.no_graph and not (world > 1 and not chain)
    graph = None
    if use_graph:
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            stack.step()            # warm every kernel/attribute before capture
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            stack.step()

    def one_step():
        if graph is not None:
            graph.replay()
        else:
            stack.step()

    sampler = ClockSampler(local_rank)
    rank_pids = [os.getpid()]
    if world > 1:
        gathered_pids = [None] * world
        dist.all_gather_object(gathered_pids, os.getpid())
        rank_pids = gathered_pids
    foreign_before = foreign_compute_processes(rank_pids) if rank == 0 else None
    if rank == 0:
        sampler.start()             # nvidia-smi needs a moment to start: sample from the warm-up on
    for _ in range(max(args.warmup, 3)):
        one_step()
    barrier()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    events[0].record()
    for i in range(args.steps):
        one_step()
        events[i + 1].record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    foreign_after = foreign_compute_processes(rank_pids) if rank == 0 else None
    elapsed_ms = events[0].elapsed_time(events[-1])
    per_step = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    alg_bytes_rank = stack.algorithmic_bytes_per_step
    alg_bytes_all = alg_bytes_rank * world
    value = alg_bytes_all / (ms_per_step / 1e3) / 1e9

    side = world == 1 and args.batch == 1 and not args.skip_batched
    per_shape = measure_shapes(device) if side else None
    batched = measure_batched(device) if side else None
    if batched is not None:
        batched["decode_step_batch8"] = measure_step_batch8(args, stack, device)
        batched["gather"] = [measure_gather(tokens, table=stack.table) for tokens in (512, 8192)]
    variants = measure_step_variants(args, stack, device) if side and chain else None

    # end-to-end through the public API with host buffers
    e2e = None
    if not args.skip_e2e:
        e2e = measure_e2e(args, stack, device, world, barrier, one_step)

    checksum = stack.checksum()
    status = stack.status()
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
        if world > 1 and chain and stack.column_sharded("o", 0):
            cfg["parallelism"] = (f"x{world}: q|k|v and gate|up sharded by rows, o and down by columns (they read what their "
                                  "own rank produced; their FP32 partial sums and the row shards travel as tagged 64-bit "
                                  "words pushed to every rank over NVLink by the chain kernel)")
        cfg["cuda_graph"] = use_graph
        gemv_launches = 1 if chain else stack.links_per_step
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "tokens_per_s": args.batch / (ms_per_step / 1e3),
            "gpu_launches": stack.launches_per_step * args.steps,
            "links_per_step": stack.links_per_step,
            "clocks": clocks,
            "parity": parity,
            "step_time_stats": sample_stats(per_step) if len(per_step) >= 5 else None,
            "foreign_compute_processes": {"before": foreign_before, "after": foreign_after},
            "roofline": {
                "bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                "frac_of_nominal_8000": per_gpu / 8000.0, "peak_source": peak_kind,
                "kernel": "tq1_gemv_chain_kernel" + (" (one launch = the whole step)" if chain else " (one launch per projection)"),
                "algorithmic_bytes_per_launch": alg_bytes_rank / gemv_launches,
                "launch_us": ms_per_step * 1e3 / gemv_launches,
                # DRAM bytes per launch: the ncu capture of the chain kernel on a 2-layer step read this ratio of
                # its algorithmic bytes; traffic grows with the units processed, so the ratio carries over.
                "traffic": (NCU_TRAFFIC_RATIO * alg_bytes_rank / gemv_launches
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
        if variants is not None:
            line["step_variants"] = variants
        if world == 1 and not args.skip_cpu_baseline:
            v, threads, reps, sec = time_cpu_layer(args.batch, budget_s=12.0, min_reps=3)
            line["cpu_baseline"] = {
                "value": v, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"one of the {args.layers} layers (7 projections, 72.3 MB packed), median of {reps} "
                          f"passes of the C restatement of the reference's NumPy decode-and-dot "
                          f"({sec * 1e3:.1f} ms per layer)",
                "numpy_restatement": time_numpy_restatement(),
            }
        print(json.dumps(line))
    graph = None        # a captured graph must not outlive the communicator whose kernels it may hold
    if world > 1:
        dist.destroy_process_group()


def time_numpy_restatement(rows: int = 1024, columns: int = 5120, budget_s: float = 4.0) -> dict:
    """The bit-equal NumPy restatement of the reference's own tq1_g128_reference_gemv
    (src/bonsai_tq1/reference.py:14-39), single core, on one k/v-sized matrix."""
    import numpy as np
    from oracle import tq1_oracle as o
    blocks, x = o.synth_matrix(rows, columns, seed=0)
    xf = x.astype(np.float32)
    times = []
    start = time.perf_counter()
    while len(times) < 2 or (time.perf_counter() - start < budget_s and len(times) < 20):
        t0 = time.perf_counter()
        o.reference_gemv(blocks, xf, rows=rows, columns=columns)
        times.append(time.perf_counter() - t0)
    med = sorted(times)[len(times) // 2]
    alg = rows * columns // 128 * 28 + 2 * (rows + columns)
    return {"value": alg / med / 1e9, "unit": UNIT, "cores": 1, "kind": "numpy-restatement",
            "sample": f"{rows}x{columns}, median of {len(times)} calls ({med * 1e3:.1f} ms each)"}


def graph_time_us(device, run, replays: int, launches: int) -> float:
    """us per launch-equivalent of `run()` captured once as a CUDA graph and replayed."""
    import torch
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
    return start.elapsed_time(stop) * 1e3 / (replays * launches)


def measure_shapes(device, ring: int = 64, replays: int = 8):
    """Batch-1 product per configured shape (the seven projection shapes, the two fused ones and 4096x4096):
    * stream: `ring` distinct weight buffers in the chunk-major panel layout (far more than L2 in total, except the smallest shapes, whose ring
      is enlarged to exceed twice L2) as independent links of one chain launch -- the HBM number;
    * warm: the same buffer `ring` times in one chain launch -- L2-resident weights;
    * launches: `ring` separate launches of the plain entry point over the distinct buffers (stream order)."""
    import ctypes
    import torch
    from ternel_b200 import _native
    from ternel_b200.chain import ChainPlan, Link, blocks_to_panels
    from ternel_b200.format import check
    from ternel_b200.stack import random_blocks_device

    lib = _native.lib()
    gen = torch.Generator(device=device)
    gen.manual_seed(77)
    shapes = [(5120, 5120), (1024, 5120), (17408, 5120), (5120, 17408), (7168, 5120), (34816, 5120), (4096, 4096)]
    out = {}
    l2 = torch.cuda.get_device_properties(device).L2_cache_size
    for n, k in shapes:
        bytes_one = n * k // 128 * 28
        count = max(ring, -(-2 * l2 // bytes_one) + 1)
        count = min(count, 256)
        weights = [random_blocks_device(n, k, gen, device) for _ in range(count)]
        x = torch.randn(k, generator=gen, device=device).to(torch.float16)
        y = torch.empty(n, dtype=torch.float16, device=device)
        ws = torch.zeros(lib.tq1_linear_workspace_bytes(1, n, k), dtype=torch.uint8, device=device)
        alg = bytes_one + 2 * (n + k)
        panels = [blocks_to_panels(w) for w in weights]
        stream_plan = ChainPlan([Link(blocks=w, panel_rows=n, x=x, y=y) for w in panels])
        warm_plan = ChainPlan([Link(blocks=panels[0], panel_rows=n, x=x, y=y) for _ in panels], workspace=stream_plan.workspace)
        canon_plan = ChainPlan([Link(blocks=w, x=x, y=y) for w in weights], workspace=stream_plan.workspace)

        def launches():
            stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
            for w in weights:
                check(lib.tq1_linear_f16(w.data_ptr(), x.data_ptr(), y.data_ptr(), 0, 1, n, k,
                                         ws.data_ptr(), ws.numel(), stream))

        us_stream = graph_time_us(device, stream_plan.run, replays, count)
        us_warm = graph_time_us(device, warm_plan.run, replays, count)
        us_canon = graph_time_us(device, canon_plan.run, replays, count)
        us_launch = graph_time_us(device, launches, replays, count)
        assert stream_plan.status() == 0
        out[f"{n}x{k}"] = {"stream_us": us_stream, "stream_gbps": alg / us_stream / 1e3,
                           "warm_l2_us": us_warm, "warm_l2_gbps": alg / us_warm / 1e3,
                           "canonical_layout_stream_us": us_canon, "canonical_layout_stream_gbps": alg / us_canon / 1e3,
                           "separate_launch_us": us_launch, "separate_launch_gbps": alg / us_launch / 1e3,
                           "ring_buffers": count, "algorithmic_bytes": alg}
        stream_plan.close(); warm_plan.close(); canon_plan.close()
        del weights, panels, stream_plan, warm_plan, canon_plan
    # sensitivity: the converted model's measured trit frequencies (35.2% / 29.7% / 35.1%)
    n, k = 34816, 5120
    weights = [blocks_to_panels(random_blocks_device(n, k, gen, device, p_zero=0.297)) for _ in range(16)]
    x = torch.randn(k, generator=gen, device=device).to(torch.float16)
    y = torch.empty(n, dtype=torch.float16, device=device)
    plan = ChainPlan([Link(blocks=w, panel_rows=n, x=x, y=y) for w in weights])
    us = graph_time_us(device, plan.run, replays, len(weights))
    out["sensitivity_real_trit_frequencies_34816x5120"] = {
        "stream_us": us, "stream_gbps": (n * k // 128 * 28 + 2 * (n + k)) / us / 1e3, "p_zero": 0.297, "ring_buffers": len(weights)}
    plan.close()
    return out


def measure_step_variants(args, stack, device, replays: int = 10):
    """The same 64-layer batch-1 step run other ways over the same resident weights: independent links (fixed
    inputs) in one chain launch, and one launch per projection."""
    import ctypes
    import torch
    from ternel_b200.chain import ChainPlan, Link
    from ternel_b200.format import check

    out = {}
    links, _ = stack.chain_links()
    scratch = {n: torch.empty(n, dtype=torch.float16, device=device) for n in {l.rows for l in links}}
    independent = [Link(blocks=l.blocks, panel_rows=l.panel_rows, x=stack.inputs[l.columns][0], y=scratch[l.rows],
                        out_scale=1.0) for l in links]
    plan = ChainPlan(independent)
    out["chain_independent_links_ms"] = graph_time_us(device, plan.run, replays, 1) / 1e3
    plan.close()
    if stack.use_panels:        # the same dependent step streaming the canonical blocks (strided 112-byte rows)
        canon, _ = stack.chain_links(panels=False)
        plan = ChainPlan(canon)
        out["chain_canonical_layout_ms"] = graph_time_us(device, plan.run, replays, 1) / 1e3
        plan.close()
    links, _ = stack.chain_links(panels=False)
    lib = stack.lib
    ws = torch.zeros(max(lib.tq1_linear_workspace_bytes(1, l.rows, l.columns) for l in links), dtype=torch.uint8, device=device)
    outs = {n: torch.empty(n, dtype=torch.float16, device=device) for n in {l.rows for l in links}}

    def separate():
        stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        for l in links:
            check(lib.tq1_linear_f16(l.blocks.data_ptr(), stack.inputs[l.columns].data_ptr(), outs[l.rows].data_ptr(), 0, 1,
                                     l.rows, l.columns, ws.data_ptr(), ws.numel(), stream))

    out["separate_launches_fixed_inputs_ms"] = graph_time_us(device, separate, replays, 1) / 1e3
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
        cases = [(m, n, k) for n, k in ((5120, 5120), (1024, 5120)) for m in (2, 4, 8, 16)]
        cases += [(m, n, k) for n, k in ((17408, 5120), (5120, 17408)) for m in (2, 4, 8, 16, 512, 2048)]
    for n, k in dict.fromkeys((n, k) for _, n, k in cases):
        l2 = torch.cuda.get_device_properties(device).L2_cache_size
        buffers = min(256, max(ring_size, -(-2 * l2 // (n * k // 128 * 28)) + 1))    # distinct weights: more than 2 x L2
        ring = [random_blocks_device(n, k, gen, device) for _ in range(buffers)]
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
                        fused=stack.fused, weights_from=stack, exchange="launches")
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
    """The same step through the public API with HOST buffers: every step copies the token ids in from pinned
    host memory and reads the result back. Chain mode: LayerStack.step (packed-embedding gather +
    ChainPlan.run, captured once as a CUDA graph) and the last projection's output; otherwise the torch custom
    ops, one call per projection, with every projection's input copied in and output copied out."""
    import torch
    import torch.distributed as dist
    from ternel_b200.ops import tq1_get_rows, tq1_matmul

    host_ids = stack.ids.cpu().pin_memory()
    if stack.exchange == "chain":
        last = stack.link_outputs[-1]
        out_host = torch.empty(last.shape, dtype=last.dtype).pin_memory()
        h2d, d2h = host_ids.numel() * 8, out_host.numel() * 2

        def step():
            stack.ids.copy_(host_ids, non_blocking=True)
            one_step()
            out_host.copy_(last, non_blocking=True)
            torch.cuda.synchronize()

        api = ("ternel_b200.stack.LayerStack.step: tq1_embedding_f16 + ternel_b200.chain.ChainPlan.run "
               "(tq1_chain_plan_run, one launch)" + (", captured once as a CUDA graph and replayed" if not args.no_graph else ""))
    else:
        host_x = {k: v.cpu().pin_memory() for k, v in stack.inputs.items()}
        keys = sorted(host_x)
        last = [(n, torch.empty((args.batch, n), dtype=torch.float16).pin_memory()) for n in sorted(stack.outputs)]
        h2d = sum(v.numel() * 2 for v in host_x.values()) + host_ids.numel() * 8
        d2h = sum(buf.numel() * 2 for _, buf in last)

        def step():
            ids = host_ids.to(device, non_blocking=True)
            dev_x = {k: host_x[k].to(device, non_blocking=True) for k in keys}
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
            for n, buf in last:
                buf.copy_(outs[n], non_blocking=True)
            torch.cuda.synchronize()

        api = "torch.ops.ternel.tq1_linear / tq1_embedding, one call per projection"

    steps = max(3, min(args.steps, 30))
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
            "steps": steps, "api": api}


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
