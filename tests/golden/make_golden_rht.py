"""Generate tests/golden/reference_golden_rht.pt.xz: the reference's quantization WITH the random
Hadamard transform (QuantizationConfig.rht), on CPU.

    python tests/golden/make_golden_rht.py /path/to/reference

The reference's PyTorch back end builds the Hadamard matrix on "cuda" by default, so this script
calls the function underneath it (fouroversix.quantize.pytorch.reference.quantize) with the same
matrix built on the CPU; everything else is the reference's own code. Inputs are seeded, small, and
stored in the fixture next to the outputs.
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
    from fouroversix.quantize.pytorch.reference import quantize as ref_quantize
    from fouroversix.quantize.utils import get_rht_matrix
    from fouroversix.utils import DataType, ScaleRule

    had = get_rht_matrix(device="cpu")
    g = torch.Generator().manual_seed(20260002)
    inputs = {
        "randn_128x256": torch.randn(128, 256, generator=g).bfloat16(),
        "grad_256x128": (torch.randn(256, 128, generator=g) * 1e-3).bfloat16(),
        "half_128x128": torch.randn(128, 128, generator=g).half(),
    }
    a = torch.randn(128, 128, generator=g)
    a[:, torch.randperm(128, generator=g)[:2]] *= 20.0
    inputs["outlier_128x128"] = a.bfloat16()
    cases = []
    for inp, x in inputs.items():
        for cfg in (dict(), dict(transpose=True), dict(scale_rule="static_6"), dict(transpose=True, scale_rule="static_6"),
                    dict(dtype="if4"), dict(transpose=True, dtype="if4"), dict(transpose=True, scale_rule="mae")):
            fmt = DataType(cfg.get("dtype", "nvfp4"))
            values, scales, amax = ref_quantize(
                x, None, had, fp4_format=fmt, scale_rule=ScaleRule(cfg.get("scale_rule", "mse")),
                transpose=cfg.get("transpose", False), use_blackwell_scale_layout=fmt == DataType.nvfp4)
            cases.append({"input": inp, "config": dict(cfg), "values": values.clone(),
                          "scale_factors": scales.view(torch.uint8).flatten().clone(), "amax": amax.reshape(1).clone()})
    buf = io.BytesIO()
    torch.save({"inputs": inputs, "cases": cases, "hadamard": had}, buf)
    out = HERE / "reference_golden_rht.pt.xz"
    out.write_bytes(lzma.compress(buf.getvalue(), preset=9))
    print(f"{len(cases)} cases, {out.stat().st_size / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
