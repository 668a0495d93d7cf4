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
192/256-row activation tiles) against the measured bf16 tensor peak, with the fraction of the
nominal dense NVFP4 peak beside it; `shapes` holds every (shape, M) case, the M <= 64 ones
timed cold from a CUDA graph over rotating weight copies against the measured HBM bandwidth;
`cpu_baseline` times the CPU restatement of the reference's kernel on this host (before any
GPU work).  `sharded`, printed last, holds the configurations that shard over GPUs: the
routed layer (T = 4096 and the decode batch, every exchange schedule, outputs checked before
they are timed), the vocabulary projection with merged per-shard candidates, and the
GPT-OSS-20B-shaped decode step (batch 64, 4096 prior tokens).  `--impl reference` times only
the CPU restatement (the reference itself is Rust behind Bazel and cannot be built here).
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


PROFILE_CASES = {
    "moe_decode64": "routed layer, 64 tokens, 32 experts, top-4 (weight-streaming expert kernels)",
    "moe_t4096": "routed layer, 4096 tokens, 32 experts, top-4 (tcgen05 grouped kernels)",
    "embedding": "packed embedding gather, 8192 rows of the 201088 x 2880 table",
    "attention": "paged-attention decode, batch 64, 4096 prior tokens, 64 query / 8 kv heads",
    "topk": "row-wise top-8 of 1024 x 201088 bf16 logits",
    "split_k": "2880->5760 linear at M=32; with --kernel-policy 2 the tcgen05 tile with K cut "
               "over a cluster of CTAs (by default the weight-streaming kernel takes it)",
    "ep_rows": "token permute and indexed k-way combine of 16384 routed rows of 2880 (T=4096)",
}


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
    parser.add_argument("--no-decode-step", action="store_true",
                        help="skip the 24-layer decode step (its weights take ~15 s to build)")
    parser.add_argument("--decode-layers", type=int, default=0,
                        help="layers of the decode step (0: all 24; fewer only for quick runs, "
                             "the record then says so)")
    parser.add_argument("--kernel-policy", type=int, default=0,
                        help="nml_nvfp4_sm100_set_kernel_policy value for this process")
    parser.add_argument("--rows", type=str, default="",
                        help="comma-separated subset of M values (profiling captures)")
    parser.add_argument("--shapes", type=str, default="",
                        help="comma-separated subset of shape names (profiling captures)")
    parser.add_argument("--case", choices=sorted(PROFILE_CASES), default="",
                        help="run only this single-GPU case `--steps` times and print its device "
                             "time (profiling captures of the kernels outside the sweep)")
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


# Nominal dense NVFP4 tensor throughput of one B200 (NVIDIA's HGX B200 datasheet figure of
# 144 PFLOP/s FP4 for 8 GPUs is with 2:4 sparsity; half of it, per GPU).  The parity-preserving
# path multiplies exact 16-bit decodes of the weights with kind::f16, so its own ceiling is the
# bf16 peak; this figure is printed beside it because the target is worded against it.
NVFP4_DENSE_TFLOPS_NOMINAL = 9000.0


def ncu_traffic(key: str):
    """dram read + write bytes per launch of a captured kernel, from the data file kept next
    to the ncu summaries (None when there is no capture for `key`)."""
    path = ROOT / "profiles" / "ncu_traffic.json"
    try:
        return json.loads(path.read_text()).get(key)
    except (OSError, ValueError):
        return None


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
        # a rank that fails in the sharded extras must not hold the others for NCCL's default
        # ten minutes
        import datetime
        dist.init_process_group("nccl", device_id=device,
                                timeout=datetime.timedelta(minutes=4))
    _abi.load()
    if args.kernel_policy:
        _abi.set_kernel_policy(args.kernel_policy)
    shapes, rows = select(args)
    full_sweep = shapes == SHAPES and rows == ROWS
    # the CPU leg runs before any GPU work, while no other thread of this process is busy
    cpu_baseline = time_cpu_baseline() if rank == 0 and world == 1 and full_sweep else None

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
        traffic = ncu_traffic("gemm_kernel_bm256_gate_up_m16384")
        roofline = {"bound": "tensor",
                    "kernel": "umma::gemm_kernel dense (launch times include the row-narrowing "
                              "passes where they run): " + ", ".join(variants),
                    "achieved": achieved, "peak": peaks["bf16_tflops_sustained"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"],
                    "frac_of_nominal_dense_nvfp4_peak": achieved / NVFP4_DENSE_TFLOPS_NOMINAL,
                    "nominal_dense_nvfp4_peak": NVFP4_DENSE_TFLOPS_NOMINAL,
                    "peak_source": f"bf16_tflops_sustained of {peaks['source']} "
                                   "(the kernel runs inside a long step); kind::f16 MMA on exact "
                                   "bf16 decodes of the NVFP4 weights",
                    "launches_per_step": len(dominant),
                    "avg_launch_ms": d_time / len(dominant) * 1e3,
                    "traffic": None if traffic is None else traffic["dram_bytes"],
                    "traffic_case": None if traffic is None else traffic["case"]}

    # wide weights with many rows take three more launches per call: two passes that narrow the
    # rows to F16 operands and the BF16-operand kernel behind the narrowed one (it returns at
    # once unless the device found the input unfit for narrowing)
    narrowed = 3 * sum(1 for c in cases if "narrowed" in selected.get(c, ("", 0))[0])
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
        "clocks": clocks, "gpu_launches": (len(cases) + narrowed) * args.steps,
        "roofline": roofline,
        "peaks": peaks,
    }

    if rank == 0 and not args.no_detail:
        line["shapes"] = shape_table(cases, durations, weights, activations, outputs, peaks,
                                     selected)
        small = [e for e in line["shapes"] if e["M"] <= 64 and e["name"] == "unembed"]
        if small:
            # the weight-streaming kernel on the one shape whose single launch is a clean HBM
            # measurement (the 2880-class weights take about a microsecond at the roofline)
            best = max(small, key=lambda e: e["frac_of_hbm_peak"])
            traffic = ncu_traffic("stream_kernel_unembed_m1")
            line["roofline_small_m"] = {
                "bound": "hbm", "kernel": f"{best['kernel']} 2880->201088 at M={best['M']}",
                "achieved": best["cold_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": best["frac_of_hbm_peak"],
                "traffic": None if traffic is None else traffic["dram_bytes"],
                "traffic_case": None if traffic is None else traffic["case"]}
    if not args.no_e2e:
        line["e2e"] = end_to_end(args, cases, weights, activations, outputs, world, barrier,
                                 flops_per_pass)
    if full_sweep and not args.no_extras:
        # free the sweep's buffers before the sharded workloads allocate theirs
        del outputs, activations
        head = weights.pop("unembed")
        weights.clear()
        torch.cuda.empty_cache()
        try:
            sharded = sharded_extras(args, rank, world, device, barrier, head, peaks)
        except Exception as error:  # noqa: BLE001 -- the sweep's line must still be printed
            sharded = {"n_gpus": world,
                       "unavailable": f"{type(error).__name__}: {error}"[:300]}
        del head
        torch.cuda.empty_cache()
        if not args.no_decode_step:
            sharded["decode_step"] = decode_step_figures(args, rank, world, device, barrier, peaks)
        if rank == 0:
            line["qkv_fused"] = qkv_fusion_figures(device)
            line["sharded"] = sharded  # last, so that it survives a truncated record
    if rank == 0:
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
            line["sharded"] = line.pop("sharded", None)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def graph_replay_ms(fn, launches_per_replay: int, repeats: int = 5):
    """Device time per call of `fn` when `launches_per_replay` calls are captured once in a
    CUDA graph and replayed: no host time between the launches.  Best of `repeats` replays."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches_per_replay):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(repeats):
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        best = min(best, begin.elapsed_time(end))
    return best / launches_per_replay


def shape_table(cases, durations, weights, activations, outputs, peaks, selected):
    """Per (shape, M) figures.  Large M: device time of the launch inside the timed region.
    M <= 64 is HBM-bound, the roofline times of the four small weights are below a launch
    latency and those weights fit in L2: these cases are timed from a CUDA graph of >= 100
    launches that rotate over distinct weight copies (>= 600 MB in total), i.e. cold from HBM
    and without host time between launches; the L2-warm graph time of one weight is kept next
    to it."""
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
            rotation = [ops.NvFp4Parameter(weight.name, weight.shape, weight.dtype,
                                           weight.payload.clone(), weight.block_scales.clone(),
                                           weight.global_scale) for _ in range(copies)]
            x, out = activations[(k, m)], outputs[(name, m)]
            state = {"next": 0}

            def one_launch():
                ops.linear(x, rotation[state["next"] % copies], out=out)
                state["next"] += 1

            launches = max(copies, -(-100 // copies) * copies)
            cold = graph_replay_ms(one_launch, launches) * 1e-3
            warm_graph = graph_replay_ms(lambda: ops.linear(x, rotation[0], out=out), 100) * 1e-3
            entry.update({"bound": "hbm", "cold_us": cold * 1e6, "cold_gbs": nbytes / cold / 1e9,
                          "frac_of_hbm_peak": nbytes / cold / 1e9 / peaks["hbm_gbs"],
                          "l2_warm_us": warm_graph * 1e6, "weight_copies": copies,
                          "timing": f"cuda graph of {launches} launches, best of 5 replays"})
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
    """Device time per replay of `fn` captured once in a CUDA graph (collectives and waits for
    other ranks included), in ms, max over ranks; None when the capture fails."""
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


def layer_check(actual, expected, mean_bar: float = 2e-3) -> dict:
    """The layer bar of the parity tests on device tensors: mean relative error <= 2e-3
    (denominator floored at 1 % of the RMS; three times that for the all-reduce schedule, which
    narrows every rank's partial sum and reduces in bf16) and the reference's own elementwise
    bound for the operator, |a - e| <= 6e-2 (1 + |e|) in bf16."""
    a, e = actual.float(), expected.float()
    floor = 0.01 * e.pow(2).mean().sqrt()
    mean_rel = ((a - e).abs() / torch_maximum(e.abs(), floor)).mean().item()
    mixed = ((a - e).abs() / (1 + e.abs())).max().item()
    return {"mean_rel": mean_rel, "max_mixed": mixed,
            "ok": bool(mean_rel <= mean_bar and mixed <= 6e-2)}


def torch_maximum(tensor, floor):
    import torch
    return torch.maximum(tensor, floor.expand_as(tensor))


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
    the GPT-OSS-20B-shaped routed layer at T = 4096 and at the decode batch of 64 (32 experts,
    top-4), expert-parallel over the job's ranks with every exchange schedule (fixed total
    work: strong scaling; efficiency = t(1) / (N t(N)) with t(1) the one-GPU layer over all
    tokens timed in the same process); the packed embedding gather (8192 rows); the 201088-wide
    unembedding at M in {1, 64, 1024}, column-sharded, as a sampler needs it (per-shard
    candidates merged) and with all logit columns gathered.  Every routed-layer schedule is
    checked on a sample of this rank's tokens against the one-GPU layer before it is timed; a
    schedule whose check fails reports `unavailable` instead of a number."""
    import torch
    import torch.distributed as dist
    from nml_b200 import expert_parallel as ep, ops, quantize
    out = {"n_gpus": world}
    generator = torch.Generator(device=device).manual_seed(99)  # same on every rank
    hidden_size, inter, experts, top_k = 2880, 2880, 32, 4

    def normal(shape, std):
        return (torch.randn(shape, device=device, generator=generator) * std).to(torch.bfloat16)

    gate_up = quantize.quantize_parameter("gate_up", normal((experts, 2 * inter, hidden_size), 0.02))
    down = quantize.quantize_parameter("down", normal((experts, hidden_size, inter), 0.02))
    gate_bias, down_bias = normal((experts, 2 * inter), 0.02), normal((experts, hidden_size), 0.02)
    router = normal((experts, hidden_size), 0.02)
    layer = ep.LocalExperts.shard(gate_up, gate_bias, down, down_bias, rank, world)
    moe_flops_per_token = 2.0 * top_k * (2 * inter * hidden_size + hidden_size * inter)
    steps = max(args.steps, 5)
    exchange = None
    for label, tokens in (("moe_t4096", 4096), ("moe_decode64", 64)):
        tokens = tokens // world * world
        x = normal((tokens, hidden_size), 1.0)
        logits = (x.float() @ router.float().t()).contiguous()  # dense router, computed once
        lo, hi = ep.shard_range(tokens, rank, world)
        x_local, logits_local = x[lo:hi].contiguous(), logits[lo:hi].contiguous()

        def single():
            return ops.routed_clamped_swiglu(x, logits, gate_up, gate_bias, down, down_bias, top_k)

        t1_eager = timed(single, 3, steps, barrier, world)
        t1_graph = timed_from_graph(single, steps, barrier, world)
        t1 = t1_graph if t1_graph is not None else t1_eager
        sample = slice(0, min(64, x_local.shape[0]))
        expected = ops.routed_clamped_swiglu(x_local[sample], logits_local[sample], gate_up,
                                             gate_bias, down, down_bias, top_k)
        record = {"tokens": tokens, "experts": experts, "top_k": top_k, "scaling": "strong",
                  "one_gpu": {"ms_per_layer": t1, "ms_eager": t1_eager,
                              "tokens_per_s": tokens / (t1 * 1e-3),
                              "tflops": moe_flops_per_token * tokens / (t1 * 1e-3) / 1e12,
                              "weight_gbs": experts * 3 * inter * hidden_size * 0.5625 /
                              (t1 * 1e-3) / 1e9},
                  "schedules": {}}
        for schedule in ("push", "alltoall", "allreduce"):
            try:
                moe = ep.ExpertParallelMoE(layer, top_k, schedule=schedule, exchange=exchange)
                result = moe(x_local, logits_local)
                torch.cuda.synchronize()
                if schedule == "push":
                    exchange = moe.exchange  # sized by the first (largest) batch, then reused
            except Exception as error:  # noqa: BLE001 -- e.g. no peer mapping on this box
                record["schedules"][schedule] = {
                    "unavailable": f"{type(error).__name__}: {error}"[:200]}
                continue
            check = layer_check(result[sample], expected,
                                6e-3 if schedule == "allreduce" and world > 1 else 2e-3)
            if world > 1:
                agreed = torch.tensor([1.0 if check["ok"] else 0.0], device=device)
                dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
                check["ok"] = bool(agreed.item() == 1.0)
            if not check["ok"]:
                record["schedules"][schedule] = {"unavailable": "output check failed", **check}
                continue
            eager = timed(lambda: moe(x_local, logits_local), 3, steps, barrier, world)
            graph = None
            if schedule != "alltoall":  # the all-to-all-v needs its split sizes on the host
                graph = timed_from_graph(lambda: moe(x_local, logits_local), steps, barrier, world)
            ms = graph if graph is not None else eager
            record["schedules"][schedule] = {
                "checked": True, "check": check, "ms_per_layer": ms, "ms_eager": eager,
                "timing": "cuda graph replay" if graph is not None else "eager launches",
                "tokens_per_s": tokens / (ms * 1e-3),
                "tflops": moe_flops_per_token * tokens / (ms * 1e-3) / 1e12,
                "per_gpu_efficiency": t1 / (world * ms)}
        out[label] = record
    del layer, gate_up, down, exchange
    torch.cuda.empty_cache()

    # packed embedding gather + column-sharded unembedding on the 201088 x 2880 table
    ids = torch.randint(0, head.shape[0], (8192,), device=device, generator=generator,
                        dtype=torch.int32)
    rows = torch.empty((8192, hidden_size), dtype=torch.bfloat16, device=device)
    ms = graph_replay_ms(lambda: ops.token_embedding(head, ids, out=rows), 20)
    gather_bytes = 8192 * (hidden_size // 2 + hidden_size // 16 + 2 * hidden_size + 4)
    out["embedding_gather"] = {"rows": 8192, "us": ms * 1e3, "gbs": gather_bytes / (ms * 1e-3) / 1e9,
                               "frac_of_hbm_peak": gather_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                               "note": "replicated per rank (rows are gathered where the token lives)"}
    sharded = ep.ShardedUnembedding(head)
    out["unembed_sharded"] = []
    for m in (1, 64, 1024):
        h = normal((m, hidden_size), 1.0)
        flops = 2.0 * m * hidden_size * head.shape[0]
        weight_bytes = head.shape[0] * hidden_size * 0.5625
        entry = {"M": m}
        for label, fn in (("top8_merged", lambda: sharded.topk(h, 8, gather_rows=False)),
                          ("all_logits", lambda: sharded(h, gather_rows=False))):
            ms = timed_from_graph(fn, 10, barrier, world)
            timing = "cuda graph replay"
            if ms is None:
                ms, timing = timed(fn, 3, 10, barrier, world), "eager launches"
            entry[label] = {"us": ms * 1e3, "tflops": flops / (ms * 1e-3) / 1e12,
                            "weight_gbs": weight_bytes / (ms * 1e-3) / 1e9, "timing": timing}
        out["unembed_sharded"].append(entry)
    return out


def decode_step_figures(args, rank, world, device, barrier, peaks) -> dict:
    """The GPT-OSS-20B-shaped decode step (24 layers, batch 64 over a KV cache of 4096 prior
    tokens per sequence, page size 16; see nml_b200/decode_step.py): tokens/s of the whole job
    and the fraction of the HBM bound of the step (packed weights touched + KV read + head).
    Non-NVFP4 operators are torch stand-ins."""
    import torch
    from nml_b200 import decode_step
    shape = decode_step.GptOssShape()
    layers = args.decode_layers or shape.layers
    batch, prior = 64, 4096
    try:
        model = decode_step.DecodeModel(shape, batch, prior, device, layers=layers)
        model.step()
        torch.cuda.synchronize()
        barrier()
        eager = timed(model.step, 2, 5, barrier, world)
        graph = timed_from_graph(model.step, 10, barrier, world)
    except Exception as error:  # noqa: BLE001
        return {"unavailable": f"{type(error).__name__}: {error}"[:300]}
    ms = graph if graph is not None else eager
    ms_full = ms * shape.layers / layers  # the head and embedding are counted once too often
    bound_bytes = shape.weight_bytes_per_step(batch, prior)
    bound_ms = bound_bytes / world / (peaks["hbm_gbs"] * 1e9) * 1e3
    return {"metric": "decode_tokens_per_s", "value": batch / (ms_full * 1e-3), "unit": "tokens/s",
            "batch": batch, "prior_tokens": prior, "layers_run": layers, "n_gpus": world,
            "ms_per_step": ms_full, "ms_eager": eager,
            "timing": "cuda graph replay" if graph is not None else "eager launches",
            "hbm_bound_ms_per_gpu": bound_ms, "frac_of_hbm_bound": bound_ms / ms_full,
            "parallelism": "single" if world == 1 else
            f"dp{world} attention, ep{world} experts (peer push), head columns / {world}",
            "stand_ins": "RMSNorm, RoPE, cache write and the bf16 router matmul are torch ops; attention, top-1 and every NVFP4 operator are this library's kernels"}


def run_case(args) -> None:
    """One small single-GPU case of a kernel the sweep does not launch, `--steps` times."""
    import torch
    from nml_b200 import _abi, ops, quantize
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the NVFP4 path has no CPU fallback")
    device = torch.device("cuda", 0)
    _abi.load()
    if args.kernel_policy:
        _abi.set_kernel_policy(args.kernel_policy)
    generator = torch.Generator(device=device).manual_seed(5)

    def normal(shape, std=0.02, dtype=torch.bfloat16):
        return (torch.randn(shape, device=device, generator=generator) * std).to(dtype)

    hidden, experts, top_k = 2880, 32, 4
    if args.case in ("moe_decode64", "moe_t4096"):
        tokens = 64 if args.case == "moe_decode64" else 4096
        gate_up = quantize.quantize_parameter("gate_up", normal((experts, 2 * hidden, hidden)))
        down = quantize.quantize_parameter("down", normal((experts, hidden, hidden)))
        gate_bias, down_bias = normal((experts, 2 * hidden)), normal((experts, hidden))
        x, logits = normal((tokens, hidden), 1.0), normal((tokens, experts), 1.0, torch.float32)

        def fn():
            ops.routed_clamped_swiglu(x, logits, gate_up, gate_bias, down, down_bias, top_k)
        nbytes = experts * 3 * hidden * hidden * 0.5625
    elif args.case == "embedding":
        rows = 201088
        table = quantize.quantize_parameter("table", normal((rows, hidden)))
        ids = torch.randint(0, rows, (8192,), device=device, generator=generator,
                            dtype=torch.int32)
        out = torch.empty((8192, hidden), dtype=torch.bfloat16, device=device)

        def fn():
            ops.token_embedding(table, ids, out=out)
        nbytes = 8192 * (hidden // 2 + hidden // 16 + 2 * hidden + 4)
    elif args.case == "attention":
        batch, prior, heads, kv_heads, dim, page = 64, 4096, 64, 8, 64, 16
        pages_per_sequence = (prior + 1 + page - 1) // page
        keys = normal((batch * pages_per_sequence, page, kv_heads, dim), 1.0)
        values = normal((batch * pages_per_sequence, page, kv_heads, dim), 1.0)
        table = torch.randperm(batch * pages_per_sequence, device=device, generator=generator) \
            .view(batch, pages_per_sequence).to(torch.int32).contiguous()
        lengths = torch.full((batch,), prior + 1, dtype=torch.int32, device=device)
        query, sinks = normal((batch, heads, dim), 1.0), normal((heads,), 1.0, torch.float32)

        def fn():
            ops.paged_attention_decode(query, keys, values, table, lengths, sinks)
        nbytes = 2 * batch * (prior + 1) * kv_heads * dim * 2
    elif args.case == "split_k":
        weight = quantize.quantize_parameter("w", normal((5760, hidden)))
        x = normal((32, hidden), 1.0)
        out = torch.empty((32, 5760), dtype=torch.bfloat16, device=device)

        def fn():
            ops.linear(x, weight, out=out)
        nbytes = linear_bytes(32, hidden, 5760)
    elif args.case == "ep_rows":
        from nml_b200 import expert_parallel as ep
        backend = ep.CudaBackend()
        tokens = 4096
        x = normal((tokens, hidden), 1.0)
        order = torch.randperm(tokens * top_k, device=device, generator=generator).to(torch.int32)
        rows_holder = {}

        def fn():
            rows_holder["rows"] = backend.gather_rows(x, order, top_k)
            backend.combine_rows(rows_holder["rows"], order.view(tokens, top_k), tokens, top_k)
        nbytes = 2 * tokens * top_k * hidden * 2 + tokens * top_k * hidden * 2 + tokens * hidden * 2
    else:
        logits = normal((1024, 201088), 1.0)

        def fn():
            ops.topk_rows(logits, 8)
        nbytes = logits.numel() * 2
    for _ in range(max(args.warmup, 3)):
        fn()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(args.steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    if _abi.device_status(0x1) != 0:
        raise RuntimeError("a kernel reported a device-side error")
    us = begin.elapsed_time(end) * 1e3 / args.steps
    print(json.dumps({"case": args.case, "what": PROFILE_CASES[args.case], "steps": args.steps,
                      "us_per_call": us, "algorithmic_bytes": nbytes,
                      "gbs": nbytes / us / 1e3, "timing": "eager launches, L2-warm where it fits"}))


def main() -> int:
    args = parse_args()
    if args.case:
        run_case(args)
        return 0
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
