"""Generate tests/golden/reference_golden_dequant32.pt.xz: the reference's `dequantize(..., intermediate_dtype=
torch.float32)` and `dequantize_values` on tensors its own PyTorch backend quantized.

    python tests/golden/make_golden_dequant32.py /path/to/reference

Stored per case: the packed tensor (values, scale factors, amax, metadata), the dequantized tensor with the
float32 intermediate in bfloat16 and float32, and the raw values (`dequantize_values`) in float16 and float32.
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
    import_reference(sys.argv[1])
    from fouroversix import QuantizationConfig, dequantize, quantize
    from fouroversix.quantize.pytorch.backend import PyTorchQuantizeBackend

    g = torch.Generator().manual_seed(20260007)
    inputs = {
        "randn_128x128": torch.randn(128, 128, generator=g).bfloat16(),
        "grad_128x128": (torch.randn(128, 128, generator=g) * 1e-3).bfloat16(),
        "ragged_100x80": torch.randn(100, 80, generator=g).bfloat16(),
    }
    z = torch.randn(128, 128, generator=g)
    z[:, torch.randperm(128, generator=g)[:2]] *= 20.0
    inputs["outlier_128x128"] = z.bfloat16()
    configs = [dict(dtype="nvfp4"), dict(dtype="nvfp4", scale_rule="static_6"), dict(dtype="if4"),
               dict(dtype="if4", scale_rule="abs_max"), dict(dtype="mxfp4", scale_rule="static_6")]
    cases = []
    for name, x in inputs.items():
        for cfg in configs:
            q = quantize(x, QuantizationConfig(backend="pytorch", **cfg))
            case = {"input": name, "config": cfg, "values": q.values.clone(),
                    "scale_factors": q.scale_factors.view(torch.uint8).clone(),
                    "amax": None if q.amax is None else q.amax.clone().reshape(-1),
                    "original_shape": tuple(q.original_shape), "padded_shape": tuple(q.padded_shape),
                    "tiled": bool(q.scale_factors_are_in_blackwell_layout),
                    "scale_rule": q.scale_rule.value}
            for out_dtype, key in ((torch.bfloat16, "dequant32_bf16"), (torch.float32, "dequant32_fp32")):
                case[key] = dequantize(q, out_dtype, backend="pytorch", intermediate_dtype=torch.float32).clone()
            case["values_fp16"] = PyTorchQuantizeBackend.dequantize_values(q, dtype=torch.float16).clone()
            case["values_fp32"] = PyTorchQuantizeBackend.dequantize_values(q, dtype=torch.float32).clone()
            cases.append(case)
    buf = io.BytesIO()
    torch.save({"inputs": inputs, "cases": cases}, buf)
    out = HERE / "reference_golden_dequant32.pt.xz"
    out.write_bytes(lzma.compress(buf.getvalue(), preset=6))
    print(f"{len(cases)} cases -> {out} ({out.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
