"""An external anchor for the FP4 GEMM numbers: cuBLASLt's NVFP4 GEMM through torch._scaled_mm, timed on the
same GPU, on the same packed operands, right beside this library's kernel.

    python baseline/scaled_mm_anchor.py [--shapes 8192x8192x8192,8192x4096x4096]

The operands are quantized once by this library (NVFP4 codes + E4M3 scales in the 128 x 4 tile order, which is
the "blocked" scale layout cuBLASLt takes), so both GEMMs read identical bytes; the per-tensor factor alpha is
applied to the library stand-in's output afterwards and is not part of its timed region. It is a stand-in for
the reference's own CUTLASS kernel (src/fouroversix/csrc/fp4_gemm.cu:40-186), which needs a CUTLASS checkout the
reference does not vendor. One GPU only: run it on its own, not under torchrun. Prints one JSON line per shape.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402


def main() -> None:
    import bench
    import fouroversix_b200 as fos
    from fouroversix_b200.matmul import B200MatmulBackend

    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="8192x8192x8192,8192x4096x4096")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    for spec in args.shapes.split(","):
        m, n, k = (int(v) for v in spec.split("x"))
        g = torch.Generator(device=dev).manual_seed(3)
        a = torch.randn(m, k, generator=g, device=dev).bfloat16()
        b = torch.randn(n, k, generator=g, device=dev).bfloat16()
        qa, qb = fos.quantize(a), fos.quantize(b)
        del a, b
        ours = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fn_ours = lambda i: B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, out=ours)  # noqa: E731
        line = {"shape": [m, n, k], "flop": 2.0 * m * n * k}

        a4 = qa.values.view(torch.float4_e2m1fn_x2)
        b4 = qb.values.view(torch.float4_e2m1fn_x2)
        sa, sb = qa.scale_factors.view(torch.float8_e4m3fn), qb.scale_factors.view(torch.float8_e4m3fn)
        lib_out = None
        try:
            fn_lib = lambda i: torch._scaled_mm(a4, b4.t(), sa, sb, out_dtype=torch.bfloat16)  # noqa: E731
            lib_out = fn_lib(0)
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001
            line["library"] = {"unavailable": f"torch._scaled_mm refused NVFP4 operands: {str(exc)[:200]}"}

        def timed(fn):
            ms = bench.time_graphs(fn, 1, args.iters, 3)
            sampler = bench.ClockSampler(0)
            sampler.start()
            t_end = time.perf_counter() + 0.5
            while time.perf_counter() < t_end:
                for i in range(20):
                    fn(i)
                torch.cuda.synchronize()
            clocks = sampler.stop()
            return {"ms": ms, "TFLOP/s": line["flop"] / (ms * 1e-3) / 1e12, "sm_mhz": clocks["sm_mhz"],
                    "ms_x_mhz": None if clocks["sm_mhz"] is None else ms * clocks["sm_mhz"], "reasons": clocks["reasons"]}

        line["fouroversix_b200"] = timed(fn_ours)
        if lib_out is not None:
            line["library"] = timed(fn_lib)
            line["library"]["what"] = "torch._scaled_mm (cuBLASLt NVFP4 block-scaled GEMM), bf16 output, alpha not applied"
            fn_ours(0)
            alpha = (qa.amax * qb.amax / (1536.0 * 1536.0)).item()
            ref = lib_out.float() * alpha
            line["max_rel_difference"] = ((ours.float() - ref).abs().max() / ref.abs().max()).item()
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
