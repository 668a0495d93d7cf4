"""Benchmark of the NVFP4 packed-weight contraction path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload (the configuration the headline metric is quoted on): the NVFP4 GEMM shape sweep
(K->N) in {2880->5120, 4096->2880, 2880->5760, 2880->2880, 2880->201088} x M in
{1, 16, 64, 512, 4096, 16384}, bf16 activations ~N(0,1), weights bf16 ~N(0, 0.02) quantized
with the NVFP4 recipe (seeded synthetic data; no public dataset is involved).  One step is one
pass over all 30 (shape, M) cases through the C ABI.  With N > 1 every rank runs the sweep on
its own replica of the weights (dense linears shard as independent replicas: weak scaling, no
data-path collective).

Prints ONE JSON line (rank 0).  `value` is whole-job TFLOP/s with inputs resident in HBM;
`e2e` is the same pass driven from pinned host buffers with the host<->device copies inside
the timed region; `roofline` describes the dominant kernel (the tcgen05 linear with its
192/256-row activation tiles) against the measured bf16 tensor peak; `cpu_baseline` times the CPU
restatement of the reference's kernel on this host.  `--impl reference` times only that CPU
restatement (the reference itself is Rust behind Bazel and cannot be built here).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

SHAPES = [("qkv", 2880, 5120), ("attn_out", 4096, 2880), ("gate_up", 2880, 5760),
          ("down", 2880, 2880), ("unembed", 2880, 201088)]
ROWS = [1, 16, 64, 512, 4096, 16384]
METRIC = "nvfp4_gemm_sweep_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "config1_nvfp4_gemm_shape_sweep(5 shapes x M in {1,16,64,512,4096,16384})"


def parse_args():
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass")
    parser.add_argument("--no-detail", action="store_true", help="skip the per-shape table")
    parser.add_argument("--no-extras", action="store_true",
                        help="skip the sharded MoE / unembedding / embedding figures")
    parser.add_argument("--graph-extras", action="store_true",
                        help="also time the expert-parallel layer replayed from a CUDA graph "
                             "(push and all-reduce schedules; removes the host time per call)")
    parser.add_argument("--kernel-policy", type=int, default=0,
                        help="nml_nvfp4_sm100_set_kernel_policy value (profiling captures: "
                             "100 + BM forces the tile height, 1000 + BM with the "
                             "shared-memory weight ring)")
    parser.add_argument("--rows", type=str, default="",
                        help="comma-separated subset of M values (profiling captures)")
    parser.add_argument("--shapes", type=str, default="",
                        help="comma-separated subset of shape names (profiling captures)")
    return parser.parse_args()


def sweep_flops(shapes, rows) -> float:
    return float(sum(2.0 * m * k * n for _, k, n in shapes for m in rows))


def linear_bytes(m: int, k: int, n: int) -> float:
    """Algorithmic bytes of one linear call: packed weights + block scales + global scale +
    activations in + outputs out."""
    return n * (k // 2) + n * (k // 16) + 4 + 2.0 * m * k + 2.0 * m * n


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"],
                "bf16_tflops_sustained": data.get("bf16_tflops_sustained", data["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append(parts + [time.time()])

    def stop(self, window_begin: float = 0.0, window_end: float = float("inf")) -> dict:
        """Summary of the samples taken inside [window_begin, window_end]; when the window
        is shorter than the sampling period, of those taken since the warm-up began."""
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.process.terminate()
        try:
            self.process.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.process.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        inside = [s for s in self.samples if window_begin <= s[-1] <= window_end]
        scope = "timed region"
        if len(inside) < 3:
            inside, scope = self.samples, "warm-up and timed region"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.samples = inside
        clocks = [int(s[0]) for s in self.samples]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names)
                   if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": int(statistics.median(clocks)), "sm_max_mhz": int(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples), "scope": scope}


# ------------------------------------------------------------------ CPU baseline

CPU_SAMPLE_ROWS = 64
CPU_SAMPLE_COLUMNS = 5760
CPU_SAMPLE_TEXT = (f"all five (K->N) shapes at M={CPU_SAMPLE_ROWS}, output columns capped at "
                   f"{CPU_SAMPLE_COLUMNS} (the first rows of each weight)")


def cpu_sample_inputs():
    """Seeded inputs of the bounded CPU sample, as numpy arrays for the oracle."""
    import numpy as np
    import torch
    from nml_b200 import quantize
    cases = []
    for index, (name, k, n) in enumerate(SHAPES):
        columns = min(n, CPU_SAMPLE_COLUMNS)
        generator = torch.Generator().manual_seed(1000 + index)
        weight = (torch.randn((columns, k), generator=generator) * 0.02).to(torch.bfloat16)
        payload, scales, g = quantize.quantize(weight)
        x = torch.randn((CPU_SAMPLE_ROWS, k), generator=generator).to(torch.bfloat16)
        cases.append((name, k, columns, x.view(torch.int16).numpy().view(np.uint16),
                      payload.numpy(), scales.numpy(), np.float32(g.item())))
    return cases


def cpu_sample_pass(cases) -> float:
    """One pass of the CPU restatement over the sample through its 16-bit handler path
    (bf16 in, f32 accumulate in the reference's order, bf16 out).  Returns flops done."""
    import oracle
    flops = 0.0
    for _, k, columns, x_bits, payload, scales, g in cases:
        oracle.linear_16(x_bits, payload, scales, g, oracle.BF16)
        flops += 2.0 * CPU_SAMPLE_ROWS * k * columns
    return flops


def time_cpu_baseline(target_seconds: float = 10.0) -> dict:
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    oracle.set_threads(cores)
    cases = cpu_sample_inputs()
    cpu_sample_pass(cases)  # warm-up
    start = time.perf_counter()
    flops = cpu_sample_pass(cases)
    once = time.perf_counter() - start
    repeats = max(1, min(200, int(target_seconds / max(once, 1e-3))))
    start = time.perf_counter()
    total = 0.0
    for _ in range(repeats):
        total += cpu_sample_pass(cases)
    elapsed = time.perf_counter() - start
    return {"value": total / elapsed / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{CPU_SAMPLE_TEXT}; {repeats} passes, {elapsed:.1f} s, OpenMP over "
                      "(row, output) pairs; the reference's own handler is single-threaded"}


def run_reference_arm(args) -> None:
    """--impl reference: the CPU restatement of the reference's NVFP4 linear on the host
    cores (the Rust reference cannot be built with the toolchain present)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    oracle.set_threads(cores)
    cases = cpu_sample_inputs()
    for _ in range(max(args.warmup, 1)):
        cpu_sample_pass(cases)
    start = time.perf_counter()
    flops = 0.0
    for _ in range(args.steps):
        flops += cpu_sample_pass(cases)
    elapsed = time.perf_counter() - start
    value = flops / elapsed / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 activations x NVFP4 (e2m1 x ue4m3) weights, f32 accumulate",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample": CPU_SAMPLE_TEXT},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": CPU_SAMPLE_TEXT + "; each step is one pass over the sample"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------- GPU arm

def select(args):
    shapes = SHAPES
    rows = ROWS
    if args.shapes:
        wanted = set(args.shapes.split(","))
        shapes = [s for s in SHAPES if s[0] in wanted]
    if args.rows:
        rows = [int(r) for r in args.rows.split(",")]
    return shapes, rows


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from nml_b200 import _abi, ops, quantize

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the NVFP4 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL prints its version banner on stdout at any NCCL_DEBUG level; the contract is
        # one JSON line on stdout.
        os.environ.pop("NCCL_DEBUG", None)
        dist.init_process_group("nccl", device_id=device)
    _abi.load()
    if args.kernel_policy:
        _abi.set_kernel_policy(args.kernel_policy)
    shapes, rows = select(args)
    full_sweep = shapes == SHAPES and rows == ROWS

    generator = torch.Generator(device=device).manual_seed(1234 + rank)
    weights = {}
    for name, k, n in shapes:
        dense = torch.empty((n, k), dtype=torch.bfloat16, device=device)
        for start in range(0, n, 32768):  # bounded f32 temporaries for the 201088-row table
            stop = min(n, start + 32768)
            dense[start:stop] = (torch.randn((stop - start, k), device=device,
                                             generator=generator) * 0.02).to(torch.bfloat16)
        weights[name] = quantize.quantize_parameter(name, dense)
        del dense
    activations = {}
    for _, k, _ in shapes:
        for m in rows:
            if (k, m) not in activations:
                activations[(k, m)] = torch.randn((m, k), device=device,
                                                  generator=generator).to(torch.bfloat16)
    outputs = {(name, m): torch.empty((m, n), dtype=torch.bfloat16, device=device)
               for name, _, n in shapes for m in rows}
    # Largest first: the host then runs far ahead of the device, so no launch waits for the
    # host, per-launch event times hold kernel time only and the clocks stay up.
    cases = sorted(((name, k, n, m) for name, k, n in shapes for m in rows),
                   key=lambda c: -(c[1] * c[2] * c[3]))
    torch.cuda.synchronize()

    selected = {}  # case -> (kernel family, activation rows per tile) the library chose

    def one_pass(events=None):
        for index, (name, k, n, m) in enumerate(cases):
            if events is not None:
                events[index][0].record()
            ops.linear(activations[(k, m)], weights[name], out=outputs[(name, m)])
            if events is not None:
                events[index][1].record()
            elif (name, k, n, m) not in selected:
                selected[(name, k, n, m)] = (_abi.last_linear_kernel(),
                                             _abi.last_linear_tile_rows())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        one_pass()
    barrier()
    if _abi.device_status(0x1) != 0:
        raise RuntimeError("a kernel reported a device-side error during warm-up")

    step_events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    for _ in cases] for _ in range(args.steps)]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    window_begin = time.time()
    begin.record()
    for step in range(args.steps):
        one_pass(step_events[step])
    end.record()
    barrier()
    clocks = sampler.stop(window_begin, time.time()) if rank == 0 else None
    elapsed_ms = begin.elapsed_time(end)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    if _abi.device_status(0x1) != 0:
        raise RuntimeError("a kernel reported a device-side error during the timed region")

    flops_per_pass = sweep_flops(shapes, rows)
    value = world * flops_per_pass * args.steps / (elapsed_ms * 1e-3) / 1e12

    # per-launch device times from the timed region (rank 0)
    durations = {}
    for index, case in enumerate(cases):
        times = [step_events[s][index][0].elapsed_time(step_events[s][index][1]) * 1e-3
                 for s in range(args.steps)]
        durations[case] = sum(times) / len(times)
    peaks = measured_peaks()
    # the dominant kernel: the tcgen05 linear with its largest activation tiles (M >= 512)
    dominant = [c for c in cases if selected.get(c, ("", 0))[1] >= 192]
    roofline = None
    if dominant:
        d_flops = sum(2.0 * m * k * n for _, k, n, m in dominant)
        d_time = sum(durations[c] for c in dominant)
        achieved = d_flops / d_time / 1e12
        variants = sorted({f"{selected[c][0]}/BM={selected[c][1]}" for c in dominant})
        roofline = {"bound": "tensor",
                    "kernel": "umma::gemm_kernel dense, bf16 operands: " + ", ".join(variants),
                    "achieved": achieved, "peak": peaks["bf16_tflops_sustained"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"],
                    "peak_source": f"bf16_tflops_sustained of {peaks['source']} "
                                   "(the kernel runs inside a long step); kind::f16 MMA on exact "
                                   "bf16 decodes of the NVFP4 weights",
                    "launches_per_step": len(dominant),
                    "avg_launch_ms": d_time / len(dominant) * 1e3,
                    "traffic": NCU_TRAFFIC["gemm_kernel_large_tiles"],
                    "traffic_case": "dram read+write bytes of one launch of 2880->5760 at "
                                    "M=16384 (algorithmic 292e6); the other launches were "
                                    "not captured"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 activations x NVFP4 (e2m1 x ue4m3) weights, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": WORKLOAD if full_sweep else
                   f"subset shapes={[s[0] for s in shapes]} rows={rows}",
                   "parallelism": f"replicas x{world}" if world > 1 else "single",
                   "l2": "one pass touches 355 MB of packed weights and 9.2 GB of outputs, "
                         "far beyond the 126 MB L2; no explicit flush"},
        "clocks": clocks, "gpu_launches": len(cases) * args.steps, "roofline": roofline,
        "peaks": peaks,
    }

    if rank == 0 and not args.no_detail:
        line["shapes"] = shape_table(cases, durations, weights, activations, outputs, peaks,
                                     selected)
    if not args.no_e2e:
        line["e2e"] = end_to_end(args, cases, weights, activations, outputs, world, barrier,
                                 flops_per_pass)
    if full_sweep and not args.no_extras:
        # free the sweep's buffers before the sharded workloads allocate theirs
        del outputs, activations
        head = weights.pop("unembed")
        weights.clear()
        torch.cuda.empty_cache()
        extras = sharded_extras(args, rank, world, device, barrier, head, peaks)
        if rank == 0:
            line.update(extras)
            line["qkv_fused"] = qkv_fusion_figures(device)
    if rank == 0:
        if world == 1 and full_sweep:
            line["cpu_baseline"] = time_cpu_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures, filled in from
# the summaries under profiles/ (None until a capture exists).
NCU_TRAFFIC = {"gemm_kernel_large_tiles": 251.7e6}  # 2880->5760 at M=16384, BM=256 (292 MB algorithmic)


def shape_table(cases, durations, weights, activations, outputs, peaks, selected):
    """Per (shape, M) figures.  Large M: device time of the launch inside the timed region.
    M <= 64 is HBM-bound and the four small weights fit in L2, so those cases are timed
    again over a rotation of distinct weight copies (>= 600 MB in total) to read them cold
    from HBM; the L2-warm time from the timed region is kept next to it."""
    import torch
    from nml_b200 import ops
    table = []
    for name, k, n, m in cases:
        flops = 2.0 * m * k * n
        nbytes = linear_bytes(m, k, n)
        warm = durations[(name, k, n, m)]
        family, tile = selected.get((name, k, n, m), ("", 0))
        entry = {"shape": f"{k}->{n}", "name": name, "M": m, "tile_rows": tile, "kernel": family,
                 "us": warm * 1e6, "tflops": flops / warm / 1e12, "gbs": nbytes / warm / 1e9}
        if m <= 64:
            weight = weights[name]
            weight_bytes = weight.payload.numel() + weight.block_scales.numel()
            copies = max(2, min(128, int(600e6 // weight_bytes) + 1))
            if weight_bytes > 300e6:
                copies = 3
            rotation = [ops.NvFp4Parameter(weight.name, weight.shape, weight.dtype,
                                           weight.payload.clone(), weight.block_scales.clone(),
                                           weight.global_scale) for _ in range(copies)]
            x, out = activations[(k, m)], outputs[(name, m)]
            for w in rotation:  # warm-up pass (also pages the copies in)
                ops.linear(x, w, out=out)
            begin = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            repeats = 3
            begin.record()
            for _ in range(repeats):
                for w in rotation:
                    ops.linear(x, w, out=out)
            end.record()
            torch.cuda.synchronize()
            cold = begin.elapsed_time(end) * 1e-3 / (repeats * copies)
            entry.update({"bound": "hbm", "cold_us": cold * 1e6, "cold_gbs": nbytes / cold / 1e9,
                          "frac_of_hbm_peak": nbytes / cold / 1e9 / peaks["hbm_gbs"],
                          "weight_copies": copies})
            del rotation
        else:
            peak = peaks["bf16_tflops_sustained"]
            entry.update({"bound": "tensor" if m >= 512 else "hbm",
                          "frac_of_bf16_peak": flops / warm / 1e12 / peak})
        table.append(entry)
    return table


def end_to_end(args, cases, weights, activations, outputs, world, barrier, flops_per_pass):
    """The same pass through the operator API from HOST buffers: every step copies each
    case's activations from pinned host memory to the device, runs the linear, and copies the
    result back to pinned host memory, all inside the timed region.  Weights stay resident on
    the device, as uploaded parameters do in the reference runtime."""
    import torch
    import torch.distributed as dist
    from nml_b200 import ops
    host_x = {key: value.cpu().pin_memory() for key, value in activations.items()}
    largest = max(out.numel() for out in outputs.values())
    host_out = torch.empty(largest, dtype=torch.bfloat16).pin_memory()
    h2d = sum(host_x[(k, m)].numel() * 2 for _, k, _, m in cases)
    d2h = sum(outputs[(name, m)].numel() * 2 for name, _, _, m in cases)

    # Three streams: uploads, kernels, downloads.  A case's kernel waits for its upload; its
    # download waits for the kernel; an activation buffer is not overwritten while a kernel
    # still reads it, an output buffer not while its previous download is in flight.
    main = torch.cuda.current_stream()
    upload, download = torch.cuda.Stream(), torch.cuda.Stream()
    x_readers_done = {key: None for key in activations}
    out_downloaded = {key: None for key in outputs}

    def one_pass():
        for name, k, n, m in cases:
            x = activations[(k, m)]
            with torch.cuda.stream(upload):
                if x_readers_done[(k, m)] is not None:
                    upload.wait_event(x_readers_done[(k, m)])
                x.copy_(host_x[(k, m)], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(upload)
            out = outputs[(name, m)]
            main.wait_event(uploaded)
            if out_downloaded[(name, m)] is not None:
                main.wait_event(out_downloaded[(name, m)])
            ops.linear(x, weights[name], out=out)
            computed = torch.cuda.Event()
            computed.record(main)
            x_readers_done[(k, m)] = computed
            with torch.cuda.stream(download):
                download.wait_event(computed)
                host_out[:out.numel()].view(m, n).copy_(out, non_blocking=True)
                done = torch.cuda.Event()
                done.record(download)
            out_downloaded[(name, m)] = done
        # the timed stream ends only when the last download has landed
        main.wait_stream(download)

    steps = max(1, min(args.steps, 5))
    one_pass()
    barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        one_pass()
    end.record()
    barrier()
    elapsed_ms = begin.elapsed_time(end)
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    return {"value": world * flops_per_pass * steps / (elapsed_ms * 1e-3) / 1e12, "unit": UNIT,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": steps,
            "ms_per_step": elapsed_ms / steps}


def timed(fn, warmup, steps, barrier, world):
    """Device time of `steps` calls of fn in ms per call, max over ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        fn()
    end.record()
    barrier()
    elapsed = begin.elapsed_time(end) / steps
    if world > 1:
        t = torch.tensor([elapsed], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t.item())
    return elapsed


def timed_from_graph(fn, steps, barrier, world):
    """Device time per replay of `fn` captured once in a CUDA graph (collectives included), in
    ms, max over ranks; None when the capture fails."""
    import torch
    import torch.distributed as dist
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            graph.replay()
        end.record()
        barrier()
        elapsed = begin.elapsed_time(end) / steps
    except Exception as error:  # noqa: BLE001 -- report and carry on with the eager figure
        print(f"cuda graph capture failed: {error}", file=sys.stderr)
        return None
    if world > 1:
        t = torch.tensor([elapsed], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t.item())
    return elapsed


def qkv_fusion_figures(device) -> list:
    """The Q/K/V projections of one GPT-OSS-20B layer (2880 -> 4096 + 512 + 512) at decode
    batch sizes: one fused launch against three linear launches (device time per layer,
    weights L2-resident; not part of `value`)."""
    import torch
    from nml_b200 import ops, quantize
    generator = torch.Generator(device=device).manual_seed(7)
    weights = [quantize.quantize_parameter(
        name, (torch.randn((n, 2880), device=device, generator=generator) * 0.02)
        .to(torch.bfloat16)) for name, n in (("q", 4096), ("k", 512), ("v", 512))]
    rows = []
    for m in (1, 16, 64):
        x = torch.randn((m, 2880), device=device, generator=generator).to(torch.bfloat16)

        def fused():
            ops.linear_qkv(x, weights[0], None, weights[1], None, weights[2], None)

        def separate():
            for w in weights:
                ops.linear(x, w)

        times = {}
        for label, fn in (("fused_us", fused), ("three_launches_us", separate)):
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(50):
                fn()
            end.record()
            torch.cuda.synchronize()
            times[label] = begin.elapsed_time(end) * 1e3 / 50
        rows.append({"M": m, **times})
    return rows


def sharded_extras(args, rank, world, device, barrier, head, peaks) -> dict:
    """Figures for the configurations that shard over GPUs (not part of `value`):
    config 2, the GPT-OSS-20B-shaped routed layer (T=4096, 32 experts, top-4), expert-parallel
    over the job's ranks with the NCCL token all-to-all (fixed total work: strong scaling);
    config 3, the packed embedding gather (8192 rows) and the 201088-wide unembedding at
    M in {1, 64, 1024} column-sharded over the ranks."""
    import torch
    from nml_b200 import expert_parallel as ep, ops, quantize
    out = {}
    generator = torch.Generator(device=device).manual_seed(99)  # same on every rank
    hidden_size, inter, experts, top_k, tokens = 2880, 2880, 32, 4, 4096

    def normal(shape, std):
        return (torch.randn(shape, device=device, generator=generator) * std).to(torch.bfloat16)

    gate_up = quantize.quantize_parameter("gate_up", normal((experts, 2 * inter, hidden_size), 0.02))
    down = quantize.quantize_parameter("down", normal((experts, hidden_size, inter), 0.02))
    gate_bias, down_bias = normal((experts, 2 * inter), 0.02), normal((experts, hidden_size), 0.02)
    router = normal((experts, hidden_size), 0.02)
    x = normal((tokens, hidden_size), 1.0)
    logits = (x.float() @ router.float().t()).contiguous()  # dense router, computed once
    lo, hi = ep.shard_range(tokens, rank, world)
    layer = ep.LocalExperts.shard(gate_up, gate_bias, down, down_bias, rank, world)
    del gate_up, down
    torch.cuda.empty_cache()
    x_local, logits_local = x[lo:hi].contiguous(), logits[lo:hi].contiguous()
    moe_flops = 2.0 * tokens * top_k * (2 * inter * hidden_size + hidden_size * inter)
    for schedule in ("alltoall", "push", "allreduce"):
        moe = ep.ExpertParallelMoE(layer, top_k, schedule=schedule)
        if schedule == "push":
            # needs every rank's buffers mapped into this process (symmetric memory); a box
            # that cannot do that gets a note instead of a number
            try:
                moe(x_local, logits_local)
                torch.cuda.synchronize()
            except Exception as error:  # noqa: BLE001
                out["moe_push"] = {"unavailable": f"{type(error).__name__}: {error}"[:200]}
                continue
        ms = timed(lambda: moe(x_local, logits_local), 3, max(args.steps, 5), barrier, world)
        graph_ms = None
        if args.graph_extras and schedule != "alltoall":  # all-to-all-v synchronises the host
            graph_ms = timed_from_graph(lambda: moe(x_local, logits_local), max(args.steps, 5),
                                        barrier, world)
        out[f"moe_{schedule}"] = {
            "ms_per_layer_from_cuda_graph": graph_ms,
            "metric": "moe_layer_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "ms_per_layer": ms, "tflops": moe_flops / (ms * 1e-3) / 1e12, "tokens": tokens,
            "experts": experts, "top_k": top_k, "n_gpus": world, "scaling": "strong",
            "schedule": schedule, "frac_of_bf16_peak":
                moe_flops / (ms * 1e-3) / 1e12 / (world * peaks["bf16_tflops_sustained"])}
    # decode-size batch (config 4's routed layer): 64 tokens
    x64, l64 = x[:64 // world * world], logits[:64 // world * world]
    lo, hi = ep.shard_range(x64.shape[0], rank, world)
    moe = ep.ExpertParallelMoE(layer, top_k, schedule="allreduce")
    ms = timed(lambda: moe(x64[lo:hi].contiguous(), l64[lo:hi].contiguous()), 3, 20, barrier,
               world)
    expert_bytes = experts * (2 * inter * hidden_size + hidden_size * inter) * 0.5625
    out["moe_decode64"] = {"metric": "moe_layer_tokens_per_s", "value": x64.shape[0] / (ms * 1e-3),
                           "unit": "tokens/s", "us_per_layer": ms * 1e3, "n_gpus": world,
                           "schedule": "allreduce",
                           "weight_gbs_if_all_experts_hit": expert_bytes / (ms * 1e-3) / 1e9}
    del layer, moe
    torch.cuda.empty_cache()

    # config 3: embedding gather + column-sharded unembedding on the 201088 x 2880 table
    ids = torch.randint(0, head.shape[0], (8192,), device=device, generator=generator,
                        dtype=torch.int32)
    rows = torch.empty((8192, hidden_size), dtype=torch.bfloat16, device=device)
    ms = timed(lambda: ops.token_embedding(head, ids, out=rows), 3, 20, barrier, world)
    gather_bytes = 8192 * (hidden_size // 2 + hidden_size // 16 + 2 * hidden_size + 4)
    out["embedding_gather"] = {"rows": 8192, "us": ms * 1e3, "gbs": gather_bytes / (ms * 1e-3) / 1e9,
                               "frac_of_hbm_peak": gather_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                               "note": "replicated per rank (rows are gathered where the token lives)"}
    sharded = ep.ShardedUnembedding(head)
    out["unembed_sharded"] = []
    for m in (1, 64, 1024):
        h = x[:m].contiguous()
        ms = timed(lambda: sharded(h, gather_rows=False), 3, 10, barrier, world)
        flops = 2.0 * m * hidden_size * head.shape[0]
        out["unembed_sharded"].append({
            "M": m, "n_gpus": world, "us": ms * 1e3, "tflops": flops / (ms * 1e-3) / 1e12,
            "weight_gbs": head.shape[0] * hidden_size * 0.5625 / (ms * 1e-3) / 1e9,
            "includes": "local linear on N/G columns + all-gather of the logit columns"})
    return out


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
