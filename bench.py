"""Benchmark of the hot path: Four-Over-Six NVFP4 quantization and the FP4 GEMM that consumes it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case quantize|dequantize|gemm [...]      (one kernel on its own, see run_case)

One JSON line on stdout (rank 0).  The primary `value` is quantize throughput in GB/s of
algorithmic traffic (2 B read + 0.5 B codes + 1/16 B scale per element) on the activation
tensor of the "quantize both operands + NVFP4 GEMM" configuration: A = 8192 x 4096 bf16,
N(0,1) with 1 % of the K-channels scaled by 20, NVFP4 with 4/6 MSE block selection.  The
`gemm` object carries the second half of the metric: FP4 GEMM TFLOP/s at M = N = K = 8192
(and the A x B^T of the same configuration).  Inputs are synthetic and seeded.

A "step" is one quantization of A (amax pass + quantize pass = 2 kernel launches), replayed
as a CUDA graph so that the Python launch cost does not hide the device time.  Four
copies of A (256 MiB) are cycled so that every step reads its input from HBM, not from
the 126 MB L2.  The `roofline` object is about the dominant kernel of a step alone, the
quantize kernel: it is launched with amax given (then the call is that one kernel), four
launches per graph replay, and its algorithmic bytes are divided by the time per launch.  Timing uses CUDA events on the stream the graphs are replayed on; with
N > 1 every rank quantizes its own A (independent stripes, no collective: weak scaling)
and the slowest rank defines the time.

`--impl reference` times the CPU restatement of the reference's PyTorch path (the oracle)
on the host cores for the same workload.
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

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

A_SHAPE = (8192, 4096)
B_SHAPE = (4096, 4096)
BYTES_PER_ELEM = 2.0 + 0.5 + 1.0 / 16.0
N_ROTATE = 4
NOMINAL_FP4_TFLOPS = 9000.0
# DRAM bytes (read + write) of one launch of the quantize kernel on the 8192x4096 tensor: a constant taken from one
# ncu capture of that kernel (67.15 MB read + 3.25 MB written; the rest of the output is still in L2 when the kernel
# ends), not something this script can measure while it runs
QUANTIZE_KERNEL_DRAM_BYTES = 70.40e6
WORKLOAD = "quantize A 8192x4096 bf16 (N(0,1), 1% K-channels x20) to NVFP4 4/6-MSE, 1x16 blocks (one A per GPU)"
CONFIG = {
    "workload": WORKLOAD,
    "l2": f"GPU arm: {N_ROTATE} rotating copies of A (256 MiB > L2) so each step reads HBM-cold input; "
          "CPU arm: one copy in host memory (64 MiB, larger than the host caches)",
}


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def make_a(seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(A_SHAPE, generator=g)
    idx = torch.randperm(A_SHAPE[1], generator=g)[: A_SHAPE[1] // 100]
    a[:, idx] *= 20.0
    return a.bfloat16()


def make_b(seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B_SHAPE, generator=g) * 0.02).bfloat16()


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def time_cuda(fn, steps: int, warmup: int) -> float:
    """Mean milliseconds per call of fn(i), CUDA events on the current stream (eager launches:
    host-side launch cost is part of the number)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def time_graphs(fn, n_variants: int, steps: int, warmup: int) -> float:
    """Mean milliseconds per step when step i is a replay of a CUDA graph that captured
    fn(i % n_variants). The kernels are short (tens of microseconds), so launching them from
    Python one by one would time the interpreter; a graph replay leaves the device work and
    the gaps between the kernels of one step. Events are recorded on the replay stream."""
    for i in range(max(n_variants, 1)):
        fn(i)
    torch.cuda.synchronize()
    graphs = []
    for i in range(n_variants):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn(i)
        graphs.append(g)
    for i in range(max(warmup, n_variants)):
        graphs[i % n_variants].replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        graphs[i % n_variants].replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def cpu_baseline_quantize(a_cpu: torch.Tensor, budget_s: float = 10.0) -> dict:
    from oracle import fos_oracle

    fos_oracle.set_num_threads(len(os.sched_getaffinity(0)))
    fos_oracle.quantize(a_cpu[:256])
    times = []
    t_end = time.perf_counter() + budget_s
    while time.perf_counter() < t_end or len(times) < 3:
        t0 = time.perf_counter()
        fos_oracle.quantize(a_cpu, dtype="nvfp4", scale_rule="mse")
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": BYTES_PER_ELEM * a_cpu.numel() / med / 1e9, "unit": "GB/s", "cores": fos_oracle.num_threads(),
            "kind": "port",
            "sample": f"full {A_SHAPE[0]}x{A_SHAPE[1]} tensor, median of {len(times)} runs of the C oracle "
                      f"(OpenMP, {fos_oracle.num_threads()} threads), {med * 1e3:.0f} ms each"}


def run_reference(args, rank: int) -> None:
    """CPU arm: the oracle (restatement of the reference's PyTorch path) on the host cores."""
    if rank != 0:
        return
    from oracle import fos_oracle

    fos_oracle.set_num_threads(len(os.sched_getaffinity(0)))   # torchrun exports OMP_NUM_THREADS=1
    a = make_a(1)
    for _ in range(max(args.warmup, 1)):
        fos_oracle.quantize(a)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fos_oracle.quantize(a, dtype="nvfp4", scale_rule="mse")
    ms = (time.perf_counter() - t0) / args.steps * 1e3
    value = BYTES_PER_ELEM * a.numel() / (ms * 1e-3) / 1e9
    threads = fos_oracle.num_threads()
    line = {
        "impl": "reference", "metric": "quantize GB/s (frac of HBM peak); FP4 GEMM TFLOP/s at 8192^3 (frac of FP4 peak)",
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": CONFIG,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "every step is one full 8192x4096 quantization by the C oracle"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import fouroversix_b200 as fos
    from fouroversix_b200.matmul import B200MatmulBackend
    from fouroversix_b200.quantize.backend import B200QuantizeBackend

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    cfg_mse = fos.QuantizationConfig(scale_rule="mse")

    a_cpu = make_a(1 + 100 * rank)
    a_sets = [a_cpu.to(dev)] + [make_a(1 + 100 * rank + 7 * i).to(dev) for i in range(1, N_ROTATE)]
    n_elem = a_cpu.numel()

    def step(i):
        return fos.quantize(a_sets[i % N_ROTATE], cfg_mse)

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = time_graphs(step, N_ROTATE, args.steps, args.warmup)
    eager_ms = time_cuda(step, args.steps, args.warmup)
    # a sustained second pass so that the clock sampler sees the kernels under load
    if rank == 0:
        t_end = time.perf_counter() + 1.0
        while time.perf_counter() < t_end:
            for i in range(50):
                step(i)
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = BYTES_PER_ELEM * n_elem * world / (ms * 1e-3) / 1e9
    modes = {}

    if rank == 0:
        # configs[0]: one 4096 x 4096 N(0,1) tensor (32 MiB: it fits on chip, and four rotating copies fit in L2)
        g1 = torch.Generator().manual_seed(0)
        c1_sets = [torch.randn(4096, 4096, generator=g1).bfloat16().to(dev) for _ in range(N_ROTATE)]
        t = time_graphs(lambda i: fos.quantize(c1_sets[i % N_ROTATE], cfg_mse), N_ROTATE, max(args.steps, 10), 3)
        modes["c1_4096x4096_mse"] = {"ms": t, "GB/s": BYTES_PER_ELEM * 4096 * 4096 / (t * 1e-3) / 1e9,
                                     "note": "whole call; 4 rotating 32 MiB inputs (128 MiB, about the size of L2)"}
        del c1_sets

    # end to end with host buffers, on every rank (each rank feeds its own GPU); the slowest rank defines the time
    if world > 1:
        dist.barrier()
    e2e_ms, serial_ms, h2d, d2h = e2e_section(args, fos, cfg_mse, a_cpu, a_sets[0])
    if world > 1:
        t = torch.tensor([e2e_ms, serial_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, serial_ms = float(t[0].item()), float(t[1].item())
    e2e_value = BYTES_PER_ELEM * n_elem * world / (e2e_ms * 1e-3) / 1e9
    e2e_serial_value = BYTES_PER_ELEM * n_elem * world / (serial_ms * 1e-3) / 1e9
    h2d, d2h = h2d * world, d2h * world

    if rank != 0:
        # the other ranks still take part in the sharded GEMM section below
        gemm_section(args, fos, B200MatmulBackend, dev, rank, world, peaks)
        stack_section(args, fos, dev, rank, world)
        return

    # the dominant kernel alone: with amax given a call is one launch of the quantize kernel
    amaxes = [x.abs().max().float().reshape(1) for x in a_sets]

    def four_kernels(_):
        for i in range(N_ROTATE):
            B200QuantizeBackend.quantize(a_sets[i], cfg_mse, amax=amaxes[i])

    kernel_ms = time_graphs(four_kernels, 1, max(args.steps, 20), 3) / N_ROTATE

    # other quantize modes of the same tensor (each: the whole call, both launches)
    for name, c in (("static_6", fos.QuantizationConfig(scale_rule="static_6")),
                    ("mse_amax_given", None),
                    ("mae", fos.QuantizationConfig(scale_rule="mae")),
                    ("abs_max", fos.QuantizationConfig(scale_rule="abs_max")),
                    ("if4_mse", fos.QuantizationConfig(dtype="if4")),
                    ("mse_2d", fos.QuantizationConfig(block_scale_2d=True)),
                    ("mse_transposed", fos.QuantizationConfig(transpose=True)),
                    ("mxfp4_static_6", fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6")),
                    ("mxfp4_static_6_transposed", fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6", transpose=True))):
        if c is None:
            fn = lambda i: B200QuantizeBackend.quantize(a_sets[i % N_ROTATE], cfg_mse, amax=amaxes[i % N_ROTATE])  # noqa: E731
        else:
            fn = lambda i, c=c: fos.quantize(a_sets[i % N_ROTATE], c)  # noqa: E731
        t = time_graphs(fn, N_ROTATE, max(args.steps, 10), 3)
        per_elem = 2.0 + 0.5 + 1.0 / 32 if name.startswith("mxfp4") else BYTES_PER_ELEM   # one scale byte per 32 values
        modes[name] = {"ms": t, "GB/s": per_elem * n_elem / (t * 1e-3) / 1e9}

    gemm = gemm_section(args, fos, B200MatmulBackend, dev, rank, world, peaks)
    stack = stack_section(args, fos, dev, rank, world)

    # the configuration as a whole: quantize both operands (activation 4/6 MSE per call, weight too)
    # and multiply, through the public front end; plus the other kernels of the path on the same tensor
    b_dev = make_b(2).to(dev)
    pipeline = {}
    t = time_graphs(lambda i: fos.quantized_matmul(a_sets[i % N_ROTATE], b_dev), N_ROTATE, max(args.steps, 10), 3)
    pipeline["quantize_both_and_multiply"] = {
        "ms": t, "shape": "A 8192x4096 @ B(4096x4096)^T",
        "note": "fouroversix_b200.quantized_matmul on two bf16 tensors: 2 x (zero, amax, quantize) + alpha + GEMM"}
    qb = fos.quantize(b_dev)
    t = time_graphs(lambda i: fos.quantized_matmul(a_sets[i % N_ROTATE], qb), N_ROTATE, max(args.steps, 10), 3)
    pipeline["quantize_activation_and_multiply"] = {"ms": t, "note": "weight quantized once, outside the timed region"}
    # static_6 activations: the same pair un-fused and with the quantization inside the GEMM (fos_gemm_nvfp4_fused_a:
    # every CTA that shares rows of A quantizes them again, n / 256 = 16 times here, so fusing costs time at this width)
    cfg_s6 = fos.QuantizationConfig(scale_rule="static_6")
    t = time_graphs(lambda i: fos.quantized_matmul(a_sets[i % N_ROTATE], qb, input_config=cfg_s6), N_ROTATE, max(args.steps, 10), 3)
    pipeline["quantize_activation_static6_and_multiply"] = {"ms": t, "note": "amax pass + quantize kernel + GEMM"}
    t = time_graphs(lambda i: fos.quantized_matmul(a_sets[i % N_ROTATE], qb, input_config=cfg_s6, fuse_input_quantization=True),
                    N_ROTATE, max(args.steps, 10), 3)
    pipeline["fused_static6_prologue_gemm"] = {"ms": t, "note": "amax pass + GEMM that quantizes its A tiles itself; same bits"}
    b_narrow = fos.quantize(make_b(2)[:256].contiguous().to(dev))
    t0 = time_graphs(lambda i: fos.quantized_matmul(a_sets[i % N_ROTATE], b_narrow, input_config=cfg_s6), N_ROTATE, max(args.steps, 10), 3)
    t1 = time_graphs(lambda i: fos.quantized_matmul(a_sets[i % N_ROTATE], b_narrow, input_config=cfg_s6, fuse_input_quantization=True),
                     N_ROTATE, max(args.steps, 10), 3)
    pipeline["fused_static6_prologue_gemm_n256"] = {"ms": t1, "unfused_ms": t0, "shape": "A 8192x4096 @ B(256x4096)^T"}
    q_sets = [fos.quantize(x, cfg_mse) for x in a_sets]
    t = time_graphs(lambda i: fos.dequantize(q_sets[i % N_ROTATE]), N_ROTATE, max(args.steps, 10), 3)
    pipeline["dequantize"] = {"ms": t, "GB/s": BYTES_PER_ELEM * n_elem / (t * 1e-3) / 1e9}
    cfg_fake = fos.QuantizationConfig(scale_rule="mse", pseudo_quantize=True)
    t = time_graphs(lambda i: fos.quantize(a_sets[i % N_ROTATE], cfg_fake), N_ROTATE, max(args.steps, 10), 3)
    pipeline["pseudo_quantize"] = {"ms": t, "GB/s": 4.0 * n_elem / (t * 1e-3) / 1e9,
                                   "note": "fused fake quantization, 2 B read + 2 B written per element"}
    del q_sets
    if world == 1:
        pipeline["experts_layer"] = experts_pipeline(dev, max(args.steps, 10))

    cpu = cpu_baseline_quantize(a_cpu) if world == 1 else None

    achieved = BYTES_PER_ELEM * n_elem / (kernel_ms * 1e-3) / 1e9
    step_rate = value / world
    line = {
        "metric": "quantize GB/s (frac of HBM peak); FP4 GEMM TFLOP/s at 8192^3 (frac of FP4 peak)",
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": CONFIG,
        "method": {
            "bytes_per_element": BYTES_PER_ELEM,
            "timing": "each step is one CUDA-graph replay of the library call (3 kernels: zero amax, amax pass, quantize); "
                      "ms_per_step_eager is the same call launched from Python",
        },
        "ms_per_step_eager": eager_ms,
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "frac_of_nominal_8TBps": achieved / 8000.0,
            "peak_source": peaks["source"],
            "kernel": "quantize_rows_mse_kernel<bf16> (the longer of the step's two kernels), launched alone "
                      "with amax given",
            "kernel_us": kernel_ms * 1e3,
            "algorithmic_bytes_per_launch": BYTES_PER_ELEM * n_elem,
            "traffic": QUANTIZE_KERNEL_DRAM_BYTES,
            "traffic_source": "a constant of this script: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of "
                              "this kernel on this tensor shape (not measured in this run)",
            "whole_step": {"achieved": step_rate, "frac": step_rate / peaks["hbm_gbs"],
                           "note": "amax pass + quantize kernel together (= value per GPU)"},
        },
        "quantize_modes": modes,
        "gemm": gemm,
        "decoder_linear_stack": stack,
        "pipeline": pipeline,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms,
                "how": "fouroversix_b200.quantize() on a staging tensor; every step copies its input from pinned host "
                       "memory and its codes, scales and amax back; steps are software-pipelined over three streams "
                       "(copy-in of step i+1 and copy-out of step i-1 overlap step i)",
                "serial_value": e2e_serial_value, "serial_ms_per_step": serial_ms},
        "gpu_launches": 3 * args.steps,
        "clocks": clocks,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    # the multi-GPU number that matters, once more and compactly at the END of the line (log tails keep it)
    line["stack_ms"] = {"n_gpus": world, "total": round(stack["ms"], 4),
                        **{k: round(v["ms"], 4) for k, v in stack["layers"].items()}}
    if "allreduce_form" in stack:
        line["stack_ms"]["allreduce_form_total"] = round(stack["allreduce_form"]["ms"], 4)
    print(json.dumps(line), flush=True)


def e2e_section(args, fos, cfg_mse, a_cpu, a_dev):
    """The metric end to end through the public API with HOST buffers: every step copies its input from pinned
    host memory, quantizes, and copies codes, scales and amax back. Returns (pipelined ms per step, serial ms per
    step, host-to-device bytes per step, device-to-host bytes per step) of this rank."""
    pinned_in = a_cpu.pin_memory()
    q0 = fos.quantize(a_dev, cfg_mse)
    host_vals = [torch.empty(q0.values.shape, dtype=torch.uint8).pin_memory() for _ in range(2)]
    host_sf = [torch.empty(q0.scale_factors.numel(), dtype=torch.uint8).pin_memory() for _ in range(2)]
    host_amax = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    staging = [torch.empty_like(a_dev) for _ in range(2)]

    # (a) one step after the other on one stream: copy in, quantize, copy out
    def e2e_step(i):
        staging[0].copy_(pinned_in, non_blocking=True)
        q = fos.quantize(staging[0], cfg_mse)
        host_vals[0].copy_(q.values, non_blocking=True)
        host_sf[0].copy_(q.scale_factors.view(torch.uint8), non_blocking=True)
        host_amax[0].copy_(q.amax, non_blocking=True)

    e2e_steps = max(4, min(args.steps, 20))
    serial_ms = time_cuda(e2e_step, e2e_steps, 2)

    # (b) the same steps software-pipelined over three streams with double buffers: the copy-in of
    # step i+1 and the copy-out of step i-1 run while step i is quantized (PCIe is full duplex).
    # Every step still copies its own input from pinned memory and its own result back.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]

    def pipelined(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(in_free[b])
                staging[b].copy_(pinned_in, non_blocking=True)
                in_ready[b].record(s_in)
            main.wait_event(in_ready[b])
            q = fos.quantize(staging[b], cfg_mse)
            in_free[b].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for t in (q.values, q.scale_factors, q.amax):
                    t.record_stream(s_out)
                host_vals[b].copy_(q.values, non_blocking=True)
                host_sf[b].copy_(q.scale_factors.view(torch.uint8), non_blocking=True)
                host_amax[b].copy_(q.amax, non_blocking=True)
                out_done[b].record(s_out)
        for b in range(2):
            main.wait_event(out_done[b])

    pipelined(4)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(main)
    pipelined(e2e_steps)
    e1.record(main)
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    h2d = a_cpu.numel() * 2
    d2h = host_vals[0].numel() + host_sf[0].numel() + 4
    return e2e_ms, serial_ms, h2d, d2h


def gemm_section(args, fos, B200MatmulBackend, dev, rank, world, peaks):
    """FP4 GEMM numbers: 8192^3 (and the 8192x4096x4096 of the configuration) on one GPU, NVFP4 and MXFP4, and the
    IF4 GEMM at the Llama-3-8B MLP shapes (4096 tokens, 4096 -> 14336 and 14336 -> 4096; fp16 tensor cores, so its
    roofline is the measured bf16 peak); with more GPUs the N dimension of B is split across ranks (column
    parallel, no collective) and the slowest rank defines the time. The GEMM runs power-limited, so every
    entry carries the median SM clock sampled while it ran and ms x MHz, which compares across boxes."""
    out = {}
    mx = fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6")
    if4 = fos.QuantizationConfig(dtype="if4")
    cases = (("square_8192", (8192, 8192, 8192), None), ("act_x_weight", (8192, 4096, 4096), None),
             ("square_8192_mxfp4", (8192, 8192, 8192), mx), ("if4_mlp_up", (4096, 14336, 4096), if4),
             ("if4_mlp_down", (4096, 4096, 14336), if4))
    for name, (m, n, k), qcfg in cases:
        n_local = n // world
        g = torch.Generator(device=dev).manual_seed(3 + rank)
        a = torch.randn(m, k, generator=g, device=dev).bfloat16()
        b = (torch.randn(n_local, k, generator=g, device=dev) * (1.0 if name.startswith("square") else 0.02)).bfloat16()
        qa, qb = (fos.quantize(a, qcfg), fos.quantize(b, qcfg)) if qcfg is not None else (fos.quantize(a), fos.quantize(b))
        d = torch.empty(m, n_local, dtype=torch.bfloat16, device=dev)
        del a, b
        fn = lambda i: B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, out=d)  # noqa: E731
        if world > 1:
            dist.barrier()
        ms = time_graphs(fn, 1, max(args.steps, 10), max(args.warmup, 3))
        clocks = None
        if rank == 0:
            # the same call back to back for half a second, so that the clock sampler sees it under load
            sampler = ClockSampler(dev.index or 0)
            sampler.start()
            t_end = time.perf_counter() + 0.5
            while time.perf_counter() < t_end:
                for i in range(20):
                    fn(i)
                torch.cuda.synchronize()
            clocks = sampler.stop()
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        tflops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        is_if4 = name.startswith("if4")
        if is_if4:
            roofline = {"bound": "tensor", "achieved": tflops / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": tflops / world / peaks["bf16_tflops"],
                        "peak_source": f"{peaks['source']} dense bf16 (the IF4 GEMM expands to fp16 and runs kind::f16 MMAs)",
                        "frac_of_nominal_2250": tflops / world / 2250.0}
        else:
            derived = NOMINAL_FP4_TFLOPS * peaks["bf16_tflops"] / 2250.0
            roofline = {"bound": "tensor", "achieved": tflops / world, "peak": NOMINAL_FP4_TFLOPS,
                        "unit": "TFLOP/s", "frac": tflops / world / NOMINAL_FP4_TFLOPS,
                        "peak_source": "nominal dense FP4 (no measured FP4 figure exists)",
                        "frac_of_bf16_scaled_peak": tflops / world / derived,
                        "bf16_scaled_peak": derived}
        out[name] = {
            "value": tflops, "unit": "TFLOP/s", "ms": ms, "m": m, "n": n, "k": k, "n_gpus": world,
            "sharding": "none" if world == 1 else f"column-parallel, N/{world} per rank, no collective",
            "roofline": roofline,
            "sm_mhz": None if clocks is None else clocks["sm_mhz"],
            "ms_x_mhz": None if clocks is None or clocks["sm_mhz"] is None else ms * clocks["sm_mhz"],
            "clock_reasons": None if clocks is None else clocks["reasons"],
            "gpu_launches_per_step": 4 if is_if4 else 2, "l2": "operands + output exceed L2",
        }
        del qa, qb, d
        torch.cuda.empty_cache()
    return out


STACK_TOKENS = 16 * 2048
HANDOFF_ROW_CHUNKS, HANDOFF_COL_CHUNKS, HANDOFF_COMM_SMS = 4, 2, 32      # settings of the row-slab hand-off in the stack
STACK_LAYERS = (  # name, parallelism, out features N, in features K: the linear layers of one Llama-3-70B decoder block
    ("qkv_proj", "column", 10240, 8192),
    ("o_proj", "row", 8192, 8192),
    ("gate_proj", "column", 28672, 8192),
    ("up_proj", "column", 28672, 8192),
    ("down_proj", "row", 8192, 28672),
)


def stack_section(args, fos, dev, rank, world):
    """The linear layers of one Llama-3-70B-shaped decoder block on 16 x 2048 tokens, tensor parallel over the
    ranks: NVFP4 4/6 weights quantized once per shard, activations quantized on every call (4/6 MSE). Every
    layer gets its own random input of the right shape (this is the stack of GEMMs, not a transformer).

    With more than one rank the layers hand activations over as ROW SLABS (sharding.TensorParallelLinear with
    scatter_output / scattered_input): a row-parallel layer reduce-scatters its partial products (chunk by
    chunk, beside the next chunk's GEMM), the column-parallel layer after it quantizes its slab with the
    ranks' common amax and all-gathers the packed slabs. `allreduce_form` times the same layers the other
    way (full activations on every rank, NCCL all-reduce after the row-parallel layers, every rank
    quantizing the whole activation). Per layer: time of the whole call, max over ranks."""
    from fouroversix_b200.sharding import TensorParallelLinear, shard_bounds

    cfg = fos.ModuleQuantizationConfig()
    steps, warm = max(5, min(args.steps, 10)), 3

    def timed(fn):
        if world > 1:
            dist.barrier()
        ms = time_cuda(lambda i: fn(), steps, warm)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def run(handoff: bool, row_chunks: int = HANDOFF_ROW_CHUNKS, col_chunks: int = HANDOFF_COL_CHUNKS, comm_sms: int = HANDOFF_COMM_SMS,
            peer_scatter: bool | None = None):
        layers, total_ms, total_flop = {}, 0.0, 0.0
        for idx, (name, mode, n, k) in enumerate(STACK_LAYERS):
            g = torch.Generator(device=dev).manual_seed(12 + idx + 100 * rank)
            if mode == "column":
                lo, hi = shard_bounds(n, rank, world, 128)
                w_shape, k_local = (hi - lo, k), k
            else:
                lo, hi = shard_bounds(k, rank, world, 64)
                w_shape, k_local = (n, hi - lo), hi - lo
            w = (torch.randn(*w_shape, generator=g, device=dev) * 0.02).bfloat16()
            rows = STACK_TOKENS // world if (handoff and mode == "column") else STACK_TOKENS
            x = torch.randn(rows, k_local, generator=g, device=dev).bfloat16()
            kw = {}
            if handoff:
                kw = dict(scattered_input=True) if mode == "column" else dict(scatter_output=True)
            if handoff:
                if mode == "row":
                    kw["peer_scatter"] = peer_scatter
                layer = TensorParallelLinear(w, cfg, mode, chunks=col_chunks if mode == "column" else row_chunks,
                                             comm_sms=comm_sms, **kw)
            else:
                layer = TensorParallelLinear(w, cfg, mode, chunks=4, **kw)
            del w
            if name == "up_proj":
                # gate_proj and up_proj read the same activation: its quantization (and gather) is counted once,
                # in gate_proj; up_proj takes the quantized activation as it is
                xq = layer.quantize_input(x)
                ms = timed(lambda: layer(xq))
                del xq
            else:
                ms = timed(lambda: layer(x))
            flop = 2.0 * STACK_TOKENS * n * k
            entry = {"mode": mode, "n": n, "k": k, "ms": ms, "TFLOP/s": flop / (ms * 1e-3) / 1e12}
            if mode == "row" and world > 1 and not handoff:
                entry["exchange"] = ("peer memory: scatter from the GEMM's epilogue, then reduce + gather by the owners"
                                     if layer._peer is not None else "NCCL all-reduce on a second stream, 4 chunks of tokens")
            layers[name] = entry
            total_ms += ms
            total_flop += flop
            del layer, x
            torch.cuda.empty_cache()
        return layers, total_ms, total_flop

    layers, total_ms, total_flop = run(handoff=world > 1)
    variants = {}
    if world > 1 and os.environ.get("FOS_STACK_VARIANTS"):
        # tuning aid: "row_chunks:col_chunks:comm_sms:peer,..." - the hand-off form with other settings, same process
        # (peer: 1 = reduce-scatter over peer memory, 0 = NCCL)
        for spec in os.environ["FOS_STACK_VARIANTS"].split(","):
            rc, cc, sm, peer = (int(v) for v in spec.split(":"))
            v_layers, v_ms, _ = run(True, rc, cc, sm, bool(peer))
            variants[spec] = {"ms": round(v_ms, 4), "layers": {k: round(v["ms"], 4) for k, v in v_layers.items()}}
    out = {
        "tokens": STACK_TOKENS, "n_gpus": world, "layers": layers, "ms": total_ms,
        "TFLOP/s": total_flop / (total_ms * 1e-3) / 1e12,
        "form": ("one GPU" if world == 1 else
                 f"row-slab hand-off: reduce-scatter after row-parallel layers (NCCL, {HANDOFF_ROW_CHUNKS} chunks beside the GEMM), common amax, "
                 "slab quantization, all-gather of packed codes + scales before column-parallel layers"),
        "how": "eager calls of sharding.TensorParallelLinear.forward (dynamic activation quantization + FP4 GEMM "
               "[+ the exchange]); CUDA events, max over ranks; weights quantized per shard outside the timed region",
    }
    if variants:
        out["variants"] = variants
    if world > 1:
        ar_layers, ar_ms, _ = run(handoff=False)
        nbytes = STACK_TOKENS * 8192 * 2
        buf = torch.empty(STACK_TOKENS, 8192, dtype=torch.bfloat16, device=dev)
        ms_ar = timed(lambda: dist.all_reduce(buf))
        half = torch.empty(STACK_TOKENS // world, 8192, dtype=torch.bfloat16, device=dev)
        ms_rs = timed(lambda: dist.reduce_scatter_tensor(half, buf))
        del buf, half
        out["allreduce_form"] = {"ms": ar_ms, "layers": {k: round(v["ms"], 4) for k, v in ar_layers.items()},
                                 "exchange": {k: v["exchange"] for k, v in ar_layers.items() if "exchange" in v}}
        out["collectives_alone"] = {
            "bytes": nbytes, "all_reduce_ms": ms_ar, "reduce_scatter_ms": ms_rs,
            "all_reduce_bus_GB/s": 2.0 * (world - 1) / world * nbytes / (ms_ar * 1e-3) / 1e9,
            "reduce_scatter_bus_GB/s": (world - 1) / world * nbytes / (ms_rs * 1e-3) / 1e9,
            "nvlink_bound_ms": {"all_reduce": 2.0 * (world - 1) / world * nbytes / 900e9 * 1e3,
                                "reduce_scatter": (world - 1) / world * nbytes / 900e9 * 1e3}}
    return out


def run_case(args) -> None:
    """One kernel of the path on its own: a few identical launches with the mean time per call (CUDA
    events), as a plain timing and as something to capture under a profiler
    (`ncu -k regex:<kernel> -s 1 -c 1 ... python bench.py --case ...`).

        --case quantize    --rows R --cols C [--rule mse|static_6|...] [--dtype nvfp4|if4|mxfp4] [--two-d]
                           [--transpose] [--amax-given] [--kernel auto|general|no_tma]
        --case dequantize  --rows R --cols C [--dtype ...]
        --case gemm        --m M --n N --k K [--dtype nvfp4|mxfp4|if4] [--variant 0|128|256|2]
        --case experts     --rows TOKENS --experts E --top-k T --k HIDDEN --n INTERMEDIATE (experts_case)

    `--graph` times replays of a CUDA graph of the call instead of launches from Python. Inputs are
    N(0,1) (the bench tensor with its outlier channels when the shape is 8192 x 4096)."""
    import fouroversix_b200 as fos
    from fouroversix_b200.matmul import B200MatmulBackend
    from fouroversix_b200.quantize.backend import B200QuantizeBackend

    dev = "cuda"

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        if args.graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            g.replay()
            torch.cuda.synchronize()
            fn = g.replay
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.iters

    if args.case in ("quantize", "dequantize"):
        rule = args.rule or ("static_6" if args.dtype == "mxfp4" else "mse")
        if (args.rows, args.cols) == A_SHAPE:
            x = make_a(1).to(dev)
        else:
            x = torch.randn(args.rows, args.cols, generator=torch.Generator().manual_seed(0)).bfloat16().to(dev)
        cfg = fos.QuantizationConfig(dtype=args.dtype, scale_rule=rule, block_scale_2d=args.two_d, transpose=args.transpose)
        amax = x.abs().max().float().reshape(1) if args.amax_given else None
        if args.case == "quantize":
            ms = timed(lambda: B200QuantizeBackend.quantize(x, cfg, amax=amax, kernel=args.kernel))
        else:
            q = fos.quantize(x, cfg)
            ms = timed(lambda: fos.dequantize(q))
        per_elem = 2.0 + 0.5 + (1.0 / 32 if args.dtype == "mxfp4" else 1.0 / 16)
        print(f"{args.case} {args.rows}x{args.cols} {args.dtype} {rule}: {ms * 1e3:.1f} us per call "
              f"({'graph replays' if args.graph else 'eager launches'}), "
              f"{per_elem * args.rows * args.cols / (ms * 1e-3) / 1e9:.0f} GB/s algorithmic")
        return
    if args.case == "experts":
        experts_case(args, timed)
        return
    rule = "static_6" if args.dtype == "mxfp4" else "mse"
    g = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn(args.m, args.k, generator=g, device=dev).bfloat16()
    b = torch.randn(args.n, args.k, generator=g, device=dev).bfloat16()
    cfg = fos.QuantizationConfig(dtype=args.dtype, scale_rule=rule)
    qa, qb = fos.quantize(a, cfg), fos.quantize(b, cfg)
    del a, b
    out = torch.empty(args.m, args.n, dtype=torch.bfloat16, device=dev)
    ms = timed(lambda: B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, out=out, variant=args.variant))
    print(f"gemm {args.m}x{args.n}x{args.k} {args.dtype} variant {args.variant}: {ms * 1e3:.1f} us per call, "
          f"{2.0 * args.m * args.n * args.k / (ms * 1e-3) / 1e12:.0f} TFLOP/s")


def experts_pipeline(dev, steps: int) -> dict:
    """The grouped experts layer (32 experts of GPT-OSS-20B shape, 4 per token, uniformly random routing) as CUDA-graph
    replays: routing tables (2 kernels), gather, 2 x (quantize, alpha, grouped GEMM), SwiGLU, combine - eleven kernels of the
    library and no read-back."""
    from fouroversix_b200.model import FourOverSixExperts

    e, h, i, top_k = 32, 2880, 2880, 4
    g = torch.Generator(device=dev).manual_seed(0)
    layer = FourOverSixExperts(
        (torch.randn(e, 2 * i, h, generator=g, device=dev) * 0.02).bfloat16(),
        (torch.randn(e, 2 * i, generator=g, device=dev) * 0.02).bfloat16(),
        (torch.randn(e, h, i, generator=g, device=dev) * 0.02).bfloat16(),
        (torch.randn(e, h, generator=g, device=dev) * 0.02).bfloat16())
    out = {"experts": e, "top_k": top_k, "hidden": h, "intermediate": i}
    for tokens in (256, 8192):
        x = torch.randn(tokens, h, generator=g, device=dev).bfloat16()
        weights, indices = torch.topk(torch.softmax(torch.randn(tokens, e, generator=g, device=dev), -1), top_k, dim=-1)
        weights = weights.bfloat16()
        ms = time_graphs(lambda _: layer(x, indices, weights), 1, steps, 3)
        out[f"tokens_{tokens}"] = {"ms": round(ms, 4), "tflops": round(2.0 * tokens * top_k * 3 * i * h / (ms * 1e-3) / 1e12, 1)}
    return out


def experts_case(args, timed) -> dict:
    """The experts of one mixture-of-experts layer (defaults: the shapes of GPT-OSS-20B, 32 experts, hidden =
    intermediate = 2880, 4 experts per token) on --rows tokens with uniformly random routing: the grouped
    launches (one quantize + one GEMM per projection, nothing read back) beside the reference's form, a host
    loop over the experts with one quantize + one GEMM each
    (src/fouroversix/model/modules/gpt_oss.py:297-335), both on this repo's kernels."""
    import fouroversix_b200 as fos
    from fouroversix_b200.model import FourOverSixExperts

    dev = "cuda"
    e, h, i, top_k, tokens = args.experts, args.k, args.n, args.top_k, args.rows
    g = torch.Generator(device=dev).manual_seed(0)
    layer = FourOverSixExperts(
        (torch.randn(e, 2 * i, h, generator=g, device=dev) * 0.02).bfloat16(),
        (torch.randn(e, 2 * i, generator=g, device=dev) * 0.02).bfloat16(),
        (torch.randn(e, h, i, generator=g, device=dev) * 0.02).bfloat16(),
        (torch.randn(e, h, generator=g, device=dev) * 0.02).bfloat16())
    x = torch.randn(tokens, h, generator=g, device=dev).bfloat16()
    weights, indices = torch.topk(torch.softmax(torch.randn(tokens, e, generator=g, device=dev), -1), top_k, dim=-1)
    weights = weights.bfloat16()
    down, gate_up = layer.quantized_weights()
    cfg = layer.config.get_activation_config()

    def loop():
        result = torch.zeros_like(x)
        mask = torch.nn.functional.one_hot(indices, num_classes=e).permute(2, 1, 0)
        for ex in range(e):
            top_k_pos, token_idx = torch.where(mask[ex])
            if token_idx.numel() == 0:
                continue
            gu = fos.quantized_matmul(x[token_idx], gate_up[ex], input_config=cfg) + layer.gate_up_proj_bias[ex]
            gate, up = gu[..., ::2].clamp(max=layer.limit), gu[..., 1::2].clamp(min=-layer.limit, max=layer.limit)
            out = fos.quantized_matmul((up + 1) * (gate * torch.sigmoid(gate * layer.alpha)), down[ex], input_config=cfg)
            result.index_add_(0, token_idx, ((out + layer.down_proj_bias[ex]) * weights[token_idx, top_k_pos, None]).to(x.dtype))
        return result

    ms_grouped = timed(lambda: layer(x, indices, weights))
    graph = args.graph
    args.graph = False                                    # the loop reads the routing back: it cannot be captured
    ms_loop = timed(loop)
    args.graph = graph
    flops = 2.0 * tokens * top_k * (2 * i * h + h * i)
    out = {"tokens": tokens, "experts": e, "top_k": top_k, "hidden": h, "intermediate": i,
           "grouped_ms": round(ms_grouped, 4), "per_expert_loop_ms": round(ms_loop, 4),
           "grouped_tflops": round(flops / (ms_grouped * 1e-3) / 1e12, 1)}
    print(f"experts {json.dumps(out)}")
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, choices=["quantize", "dequantize", "gemm", "experts", "stack"], help="one kernel on its own (run_case)")
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--rows", type=int, default=A_SHAPE[0])
    ap.add_argument("--cols", type=int, default=A_SHAPE[1])
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--rule", default=None)
    ap.add_argument("--dtype", default="nvfp4")
    ap.add_argument("--two-d", action="store_true")
    ap.add_argument("--transpose", action="store_true")
    ap.add_argument("--amax-given", action="store_true")
    ap.add_argument("--kernel", default="auto", choices=["auto", "general", "no_tma"])
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--graph", action="store_true")
    args = ap.parse_args()
    side = 2880 if args.case == "experts" else 8192          # default m, n, k of the case
    args.m, args.n, args.k = (v if v is not None else side for v in (args.m, args.n, args.k))
    if args.case == "stack":
        # the decoder stack on its own (under torchrun for more than one GPU): python -m torch.distributed.run
        # --nproc-per-node N bench.py --case stack
        import fouroversix_b200 as fos

        rank, world, local_rank = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=dev)
        try:
            out = stack_section(args, fos, dev, rank, world)
            if rank == 0:
                print(json.dumps(out))
        finally:
            if world > 1:
                dist.barrier()
                dist.destroy_process_group()
        return
    if args.case is not None:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the GPU path has no CPU fallback")
        run_case(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU path has no CPU fallback")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
