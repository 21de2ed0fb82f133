"""Generate tests/golden/reference_golden.pt.xz by running the reference project's own PyTorch backend.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference package is imported straight from its `src/` directory (its
`__init__` asks importlib.metadata for an installed version, so that one call is
answered here).  Inputs are seeded, small, and stored in the fixture next to the
reference's outputs, so the fixtures do not depend on the random generator of the
machine that later reads them.
"""

from __future__ import annotations

import importlib.metadata as md
import io
import lzma
import sys
import warnings
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent


def import_reference(root: str):
    orig = md.version
    md.version = lambda name: "1.1.0" if name == "fouroversix" else orig(name)
    warnings.filterwarnings("ignore")
    sys.path.insert(0, str(Path(root) / "src"))
    import fouroversix  # noqa: PLC0415

    return fouroversix


def make_inputs() -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(20260001)
    x = {}
    x["randn_128x128"] = torch.randn(128, 128, generator=g).bfloat16()
    x["randn_256x128"] = torch.randn(256, 128, generator=g).bfloat16()
    a = torch.randn(128, 128, generator=g)
    a[:, torch.randperm(128, generator=g)[:2]] *= 20.0
    x["outlier_128x128"] = a.bfloat16()
    x["weight_128x128"] = (torch.randn(128, 128, generator=g) * 0.02).bfloat16()
    z = torch.randn(128, 128, generator=g)
    c = (torch.randn(4, 128, 128, generator=g) ** 2).sum(0)
    x["student_128x128"] = (0.5 * z / (c / 4).sqrt()).bfloat16()
    x["grad_128x128"] = (torch.randn(128, 128, generator=g) * 1e-3).bfloat16()
    x["half_128x64"] = torch.randn(128, 64, generator=g).half()
    x["ragged_100x80"] = torch.randn(100, 80, generator=g).bfloat16()
    x["zeros_128x64"] = torch.zeros(128, 64, dtype=torch.bfloat16)
    x["ones_128x64"] = torch.ones(128, 64, dtype=torch.bfloat16)
    x["rand01_128x64"] = torch.rand(128, 64, generator=g).bfloat16()
    e = torch.zeros(128, 64, dtype=torch.bfloat16)
    e[0, :16] = torch.tensor([6, -6, 0.25, -0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.0, -0.01, 0.01, 3.0, 4.0, 1.0])
    e[1, :16] = torch.tensor([1e-3] * 8 + [-1e-3] * 8)
    e[2, :16] = torch.tensor([3.0, -3.0] * 8)
    e[3, 16:32] = torch.tensor([0.0, -0.0] * 8)
    e[4, :16] = torch.tensor([2.0 ** -130] * 16)          # bf16 subnormals
    e[5, :16] = torch.linspace(-6, 6, 16)
    x["edges_128x64"] = e
    return x


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref_root = sys.argv[1]
    fos = import_reference(ref_root)
    from fouroversix import QuantizationConfig, dequantize, quantize, quantized_matmul

    inputs = make_inputs()
    cases = []

    def run(name, inp, **cfg):
        x = inputs[inp]
        q = quantize(x, QuantizationConfig(backend="pytorch", **cfg))
        case = {
            "name": name, "input": inp, "config": dict(cfg),
            "values": q.values.clone(),
            "scale_factors": q.scale_factors.contiguous().view(torch.uint8).flatten().clone(),
            "amax": q.amax.clone().reshape(1),
            "original_shape": tuple(q.original_shape), "padded_shape": tuple(q.padded_shape),
            "tiled": bool(q.scale_factors_are_in_blackwell_layout),
        }
        if not cfg.get("transpose") and cfg.get("scale_rule") in {"mse", "static_6", "static_4"}:
            case["dequant_bf16"] = dequantize(q, torch.bfloat16, backend="pytorch").clone()
        if inp in {"randn_256x128", "half_128x64"}:
            case["dequant_fp32"] = dequantize(q, torch.float32, backend="pytorch").clone()
            case["dequant_fp16"] = dequantize(q, torch.float16, backend="pytorch").clone()
        cases.append(case)
        return q

    nv_rules = ["static_6", "static_4", "mse", "mae", "abs_max"]
    if_rules = ["mse", "mae", "abs_max"]
    bulk = ["randn_128x128", "outlier_128x128", "weight_128x128", "student_128x128", "grad_128x128"]
    for inp in bulk:
        for rule in nv_rules:
            for two_d in (False, True):
                for tr in (False, True):
                    run(f"nvfp4-{rule}-{'2d' if two_d else '1d'}-{'t' if tr else 'n'}-{inp}", inp,
                        dtype="nvfp4", scale_rule=rule, block_scale_2d=two_d, transpose=tr)
        for rule in if_rules:
            for two_d in (False, True):
                for tr in (False, True):
                    run(f"if4-{rule}-{'2d' if two_d else '1d'}-{'t' if tr else 'n'}-{inp}", inp,
                        dtype="if4", scale_rule=rule, block_scale_2d=two_d, transpose=tr)
    for rule in ["static_6", "mse"]:
        for tr in (False, True):
            run(f"nvfp4-{rule}-1d-{'t' if tr else 'n'}-randn_256x128", "randn_256x128",
                dtype="nvfp4", scale_rule=rule, transpose=tr)
    for inp in ["half_128x64", "ragged_100x80", "zeros_128x64", "ones_128x64", "rand01_128x64", "edges_128x64"]:
        for rule in ["static_6", "mse"]:
            run(f"nvfp4-{rule}-1d-n-{inp}", inp, dtype="nvfp4", scale_rule=rule)
        run(f"if4-mse-1d-n-{inp}", inp, dtype="if4", scale_rule="mse")
        run(f"nvfp4-mse-2d-n-{inp}", inp, dtype="nvfp4", scale_rule="mse", block_scale_2d=True)

    # matmul: pytorch backend = bf16(deq32(a) @ deq32(b).T); alpha as the CUTLASS backend builds it
    mm = []
    g = torch.Generator().manual_seed(20260002)
    for (m, n, k), cfg_a, cfg_b in [
        ((128, 128, 128), dict(), dict()),
        ((256, 128, 192), dict(scale_rule="static_6"), dict(scale_rule="static_6")),
        ((128, 256, 128), dict(), dict(scale_rule="static_4")),
        ((100, 72, 80), dict(), dict()),
        ((128, 128, 128), dict(dtype="if4"), dict(dtype="if4")),
        ((128, 128, 256), dict(block_scale_2d=True), dict(transpose=False)),
    ]:
        a = torch.randn(m, k, generator=g).bfloat16()
        b = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
        qa = quantize(a, QuantizationConfig(backend="pytorch", **cfg_a))
        qb = quantize(b, QuantizationConfig(backend="pytorch", **cfg_b))
        out = quantized_matmul(qa, qb, backend="pytorch")
        out32 = quantized_matmul(qa, qb, backend="pytorch", out_dtype=fos.DataType.float32)
        qt = qa.dtype.quantized_value_type
        alpha = (qa.amax * qb.amax) / (
            qt.get_maximum_value(qa.scale_rule) * qa.dtype.scale_type.get_maximum_value(qa.scale_rule)
            * qb.dtype.quantized_value_type.get_maximum_value(qb.scale_rule)
            * qb.dtype.scale_type.get_maximum_value(qb.scale_rule)
            * qa.round_style.adjustment_factor * qb.round_style.adjustment_factor
        )
        mm.append({"a": a, "b": b, "cfg_a": cfg_a, "cfg_b": cfg_b, "out_bf16": out.clone(),
                   "out_fp32": out32.clone(), "alpha": alpha.to(torch.float32).reshape(1).clone()})

    buf = io.BytesIO()
    torch.save({"inputs": inputs, "cases": cases, "matmul": mm,
                "reference_version": "1.1.0", "torch_version": torch.__version__}, buf)
    out = HERE / "reference_golden.pt.xz"
    out.write_bytes(lzma.compress(buf.getvalue(), preset=6))
    size = out.stat().st_size
    print(f"wrote {len(cases)} quantize cases, {len(mm)} matmul cases, {size / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
