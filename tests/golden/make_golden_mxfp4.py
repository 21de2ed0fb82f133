"""Generate tests/golden/reference_golden_mxfp4.pt.xz: the reference's MXFP4 path (E8M0 scale per
32 values, no per-tensor scale) on CPU: quantize, dequantize and the PyTorch matmul.

    python tests/golden/make_golden_mxfp4.py /path/to/reference

Inputs are seeded, small, and stored in the fixture next to the outputs. Transposed cases use
shapes that need no padding (the reference pads before it transposes).
"""

from __future__ import annotations

import io
import lzma
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

from make_golden import import_reference  # noqa: E402


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    import_reference(sys.argv[1])
    from fouroversix import QuantizationConfig, dequantize, quantize, quantized_matmul
    from fouroversix.utils import DataType

    g = torch.Generator().manual_seed(20260003)
    inputs = {
        "randn_128x256": torch.randn(128, 256, generator=g).bfloat16(),
        "weight_256x128": (torch.randn(256, 128, generator=g) * 0.02).bfloat16(),
        "grad_128x128": (torch.randn(128, 128, generator=g) * 1e-3).bfloat16(),
        "half_128x128": torch.randn(128, 128, generator=g).half(),
        "ragged_100x200": torch.randn(100, 200, generator=g).bfloat16(),
        "zeros_128x128": torch.zeros(128, 128, dtype=torch.bfloat16),
    }
    a = torch.randn(128, 128, generator=g)
    a[:, torch.randperm(128, generator=g)[:2]] *= 20.0
    inputs["outlier_128x128"] = a.bfloat16()
    e = torch.zeros(128, 128, dtype=torch.bfloat16)
    e[0, :32] = torch.tensor([6, -6, 0.25, -0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.0, -0.01, 0.01, 3.0, 4.0, 1.0] * 2)
    e[1, :32] = torch.tensor([3.0, -3.0] * 16)            # max / 6 is a power of two: the exponent is not rounded up
    e[2, :32] = torch.tensor([2.0 ** -130] * 32)          # bf16 subnormals
    e[3, :32] = torch.linspace(-5, 5, 32)
    e[4, 32:64] = torch.tensor([1e30, -1e-30] * 16)
    e[5, :32] = torch.tensor([4.0, 0.3] * 16)
    inputs["edges_128x128"] = e
    cases = []
    for inp, x in inputs.items():
        for cfg in (dict(scale_rule="static_6"), dict(scale_rule="static_4"), dict(scale_rule="static_6", transpose=True),
                    dict(scale_rule="static_6", block_scale_2d=True)):
            if cfg.get("transpose") and inp.startswith("ragged"):
                continue
            q = quantize(x, QuantizationConfig(dtype="mxfp4", backend="pytorch", **cfg))
            case = {"input": inp, "config": dict(cfg), "values": q.values.clone(),
                    "scale_factors": q.scale_factors.view(torch.uint8).flatten().clone(), "amax": q.amax.reshape(1).clone(),
                    "original_shape": tuple(q.original_shape), "padded_shape": tuple(q.padded_shape), "dequantized": {}}
            for name, dt in (("bfloat16", torch.bfloat16), ("float16", torch.float16), ("float32", torch.float32)):
                case["dequantized"][name] = dequantize(q, dt).clone()
            cases.append(case)
    matmuls = []
    cfg = QuantizationConfig(dtype="mxfp4", scale_rule="static_6", backend="pytorch")
    for a_name, b_name in (("randn_128x256", "randn_128x256"), ("grad_128x128", "outlier_128x128"), ("half_128x128", "weight_256x128")):
        qa, qb = quantize(inputs[a_name], cfg), quantize(inputs[b_name], cfg)
        for name, dt in (("bfloat16", "bfloat16"), ("float32", "float32")):
            matmuls.append({"a": a_name, "b": b_name, "out_dtype": name,
                            "out": quantized_matmul(qa, qb, backend="pytorch", out_dtype=DataType(dt)).clone()})
    buf = io.BytesIO()
    torch.save({"inputs": inputs, "cases": cases, "matmuls": matmuls}, buf)
    out = HERE / "reference_golden_mxfp4.pt.xz"
    out.write_bytes(lzma.compress(buf.getvalue(), preset=9))
    print(f"{len(cases)} quantize cases, {len(matmuls)} matmul cases, {out.stat().st_size / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
