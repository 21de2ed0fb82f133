"""Small, self-contained launches of each kernel, meant to be run under a profiler.

    python -m fouroversix_b200.profile_cases quantize --rows 8192 --cols 8192 --rule mse [--amax-given]
    python -m fouroversix_b200.profile_cases dequantize --rows 8192 --cols 8192
    python -m fouroversix_b200.profile_cases gemm --m 4096 --n 4096 --k 4096 [--variant 0|128|256|2] [--debug BITS] [--graph]
    python -m fouroversix_b200.profile_cases gemm-if4 --m 4096 --n 4096 --k 4096

Each case allocates its inputs, runs the call `--iters` times (default 6) and prints the mean
time per call measured with CUDA events, so the same command gives a plain timing without a
profiler and a few identical launches to capture with one (`ncu -k regex:<kernel> -s 2 -c 2`).
Inputs are larger than the 126 MB L2 when the default sizes are kept for quantize.
`--graph` times replays of a CUDA graph of the call instead of launches from Python (the
kernels are short). `--debug BITS` sets the GEMM's timing-experiment bits (1: no scale copies,
2: no operand loads, 4: no output stores, 16: no MMAs; the RESULT IS WRONG with any of them):
switching parts off one at a time shows what each costs.
"""

from __future__ import annotations

import argparse

import torch

import fouroversix_b200 as fos
from fouroversix_b200 import _native
from fouroversix_b200.matmul import B200MatmulBackend
from fouroversix_b200.quantize.backend import B200QuantizeBackend


def _timed(fn, iters: int, graph: bool = False) -> float:
    fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        g.replay()
        torch.cuda.synchronize()
        fn = g.replay
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["quantize", "dequantize", "gemm", "gemm-if4"])
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--rule", default="mse")
    ap.add_argument("--dtype", default="nvfp4")
    ap.add_argument("--two-d", action="store_true")
    ap.add_argument("--transpose", action="store_true")
    ap.add_argument("--amax-given", action="store_true")
    ap.add_argument("--exact-only", action="store_true")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--debug", type=int, default=0)
    ap.add_argument("--graph", action="store_true")
    args = ap.parse_args()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)

    if args.case in ("quantize", "dequantize"):
        x = torch.randn(args.rows, args.cols, generator=g, device=dev).bfloat16()
        cfg = fos.QuantizationConfig(dtype=args.dtype, scale_rule=args.rule, block_scale_2d=args.two_d,
                                     transpose=args.transpose)
        amax = x.abs().max().float().reshape(1) if args.amax_given else None
        if args.case == "quantize":
            ms = _timed(lambda: B200QuantizeBackend.quantize(x, cfg, amax=amax, exact_only=args.exact_only), args.iters, args.graph)
        else:
            q = fos.quantize(x, cfg)
            ms = _timed(lambda: fos.dequantize(q), args.iters, args.graph)
        gbs = 2.5625 * args.rows * args.cols / (ms * 1e-3) / 1e9
        print(f"{args.case} {args.rows}x{args.cols} {args.dtype} {args.rule}: {ms * 1e3:.1f} us per call "
              f"({'graph replays' if args.graph else 'eager launches'}), {gbs:.0f} GB/s algorithmic")
        return

    dtype = "if4" if args.case == "gemm-if4" else args.dtype
    rule = "static_6" if dtype == "mxfp4" else "mse"
    a = torch.randn(args.m, args.k, generator=g, device=dev).bfloat16()
    b = torch.randn(args.n, args.k, generator=g, device=dev).bfloat16()
    qa = fos.quantize(a, fos.QuantizationConfig(dtype=dtype, scale_rule=rule))
    qb = fos.quantize(b, fos.QuantizationConfig(dtype=dtype, scale_rule=rule))
    out = torch.empty(args.m, args.n, dtype=torch.bfloat16, device=dev)
    _native.lib().fos_set_option(1, args.variant)
    _native.check(_native.lib().fos_set_option(2, args.debug), "fos_set_option")
    try:
        ms = _timed(lambda: B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, out=out),
                    args.iters, args.graph)
    finally:
        _native.lib().fos_set_option(1, 0)
        _native.lib().fos_set_option(2, 0)
    print(f"{args.case} {args.m}x{args.n}x{args.k} variant {args.variant} debug {args.debug}: {ms * 1e3:.1f} us per call, "
          f"{2.0 * args.m * args.n * args.k / (ms * 1e-3) / 1e12:.0f} TFLOP/s")


if __name__ == "__main__":
    main()
