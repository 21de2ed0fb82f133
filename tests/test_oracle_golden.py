"""Pin the CPU oracle to the reference: every golden vector must match byte for byte.

The vectors in tests/golden/reference_golden.pt.xz were produced by the reference's
own PyTorch backend (tests/golden/make_golden.py).  They cover all five scale rules,
1-D and 16x16 blocks, transposed quantization, NVFP4 and IF4, bf16 and fp16 inputs,
ragged shapes, all-zero input and hand-made rounding ties.
"""

from __future__ import annotations

import torch


def _run(oracle, golden, case):
    x = golden["inputs"][case["input"]]
    cfg = case["config"]
    return oracle.quantize(
        x, dtype=cfg.get("dtype", "nvfp4"), scale_rule=cfg.get("scale_rule", "mse"),
        block_scale_2d=cfg.get("block_scale_2d", False), transpose=cfg.get("transpose", False))


def test_quantize_matches_reference_bytes(oracle, golden):
    bad = []
    for case in golden["cases"]:
        q = _run(oracle, golden, case)
        assert q.padded_shape == tuple(case["padded_shape"]), case["name"]
        assert q.original_shape == tuple(case["original_shape"]), case["name"]
        assert q.tiled == case["tiled"], case["name"]
        n_val = int((q.values != case["values"]).sum())
        n_sf = int((q.scale_factors != case["scale_factors"]).sum())
        same_amax = torch.equal(q.amax, case["amax"])
        if n_val or n_sf or not same_amax:
            bad.append((case["name"], n_val, n_sf, same_amax))
        # the saturating hardware conversion and the reference's unclamped rounding agree below 7
        assert q.worst_scaled < 7.0, case["name"]
    assert not bad, bad[:10]


def test_dequantize_matches_reference_bits(oracle, golden):
    checked = 0
    for case in golden["cases"]:
        for key, dt in (("dequant_bf16", torch.bfloat16), ("dequant_fp16", torch.float16),
                        ("dequant_fp32", torch.float32)):
            if key not in case:
                continue
            cfg = case["config"]
            out = oracle.dequantize_raw(
                case["values"], case["scale_factors"], case["amax"], cfg.get("dtype", "nvfp4"),
                cfg.get("scale_rule", "mse"), tuple(case["original_shape"]), dt, tiled=case["tiled"])
            ref = case[key]
            view = torch.int32 if dt == torch.float32 else torch.int16
            assert torch.equal(out.view(view), ref.contiguous().view(view)), (case["name"], key)
            checked += 1
    assert checked > 60


def test_matmul_and_alpha_match_reference(oracle, golden):
    for mm in golden["matmul"]:
        ca, cb = mm["cfg_a"], mm["cfg_b"]
        qa = oracle.quantize(mm["a"], dtype=ca.get("dtype", "nvfp4"), scale_rule=ca.get("scale_rule", "mse"),
                             block_scale_2d=ca.get("block_scale_2d", False))
        qb = oracle.quantize(mm["b"], dtype=cb.get("dtype", "nvfp4"), scale_rule=cb.get("scale_rule", "mse"))
        assert oracle.alpha(qa, qb) == mm["alpha"].item()
        out32 = oracle.matmul(qa, qb, torch.float32)
        ref32 = mm["out_fp32"]
        # fp32 accumulation order differs between sgemm implementations: tolerance, not bits
        denom = ref32.abs().max().clamp_min(1e-30)
        assert ((out32 - ref32).abs().max() / denom).item() < 1e-5
        out16 = oracle.matmul(qa, qb, torch.bfloat16)
        frac = (out16 != mm["out_bf16"]).float().mean().item()
        assert frac <= 1e-3, frac          # the reference's own cross-backend criterion


def test_division_shortcut_used_by_the_kernels_is_exact(oracle):
    """bmax / 6 via multiply + two FMAs equals the IEEE quotient for every bf16 and fp16 value."""
    import ctypes
    fn = oracle.lib().fos_oracle_check_div6
    fn.restype = ctypes.c_long
    assert fn() == 0


def test_division_free_quotient_of_the_dequantize_kernel_is_exact(oracle):
    """(value * amax) / divisor is computed as a quotient estimate, an exact remainder and one
    correction. Compared here with the IEEE quotient for every 61st finite binary32 numerator with
    |a| >= 2^-100 and each of the three divisors; the same function with stride 1 is the exhaustive
    check (0 mismatches for |a| >= 2^-100, about two minutes on eight cores)."""
    import ctypes
    fn = oracle.lib().fos_oracle_check_div_const
    fn.restype = ctypes.c_int64
    fn.argtypes = [ctypes.c_float, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float]
    for d in (1536.0, 1792.0, 2688.0):
        assert fn(d, 3, 61, 2.0 ** -100) == 0
    # and the guard is needed: below it the remainder underflows and the sequence can be off
    assert fn(1536.0, 5, 1021, 0.0) > 0


def test_oracle_reproduces_the_reference_with_the_hadamard_transform(oracle):
    """Quantization behind the 16-point random Hadamard transform (QuantizationConfig.rht), plain and
    transposed, NVFP4 and IF4: codes, scales and amax equal the reference's, byte for byte."""
    import io
    import lzma
    from pathlib import Path

    raw = lzma.decompress((Path(__file__).parent / "golden" / "reference_golden_rht.pt.xz").read_bytes())
    gold = torch.load(io.BytesIO(raw), weights_only=False)
    assert len(gold["cases"]) >= 28
    for case in gold["cases"]:
        x = gold["inputs"][case["input"]]
        got = oracle.quantize(x, rht=True, **case["config"])
        v = case["values"]
        assert torch.equal(got.values[: v.shape[0], : v.shape[1]], v), (case["input"], case["config"])
        n = case["scale_factors"].numel()
        assert torch.equal(got.scale_factors[:n], case["scale_factors"]), (case["input"], case["config"])
        assert torch.equal(got.amax.reshape(1), case["amax"]), (case["input"], case["config"])


def _load_golden(name: str):
    import io
    import lzma
    from pathlib import Path

    raw = lzma.decompress((Path(__file__).parent / "golden" / name).read_bytes())
    return torch.load(io.BytesIO(raw), weights_only=False)


def test_oracle_reproduces_the_reference_for_mxfp4(oracle):
    """MXFP4 (E8M0 scale per 32 values, static rules): codes, scales, the dequantized tensors in three
    output types (bit for bit) and the PyTorch matmul of the reference."""
    gold = _load_golden("reference_golden_mxfp4.pt.xz")
    assert len(gold["cases"]) >= 31
    for case in gold["cases"]:
        x = gold["inputs"][case["input"]]
        tag = (case["input"], case["config"])
        got = oracle.quantize(x, dtype="mxfp4", **case["config"])
        assert got.padded_shape == case["padded_shape"] and got.original_shape == case["original_shape"], tag
        assert torch.equal(got.values, case["values"]), tag
        assert torch.equal(got.scale_factors, case["scale_factors"]), tag
        assert torch.equal(got.amax, case["amax"]), tag
        assert got.worst_scaled <= 6.0, tag
        for name, ref in case["dequantized"].items():
            dt = getattr(torch, name)
            out = oracle.dequantize(got, dt)
            view = torch.int32 if dt == torch.float32 else torch.int16
            assert torch.equal(out.view(view), ref.contiguous().view(view)), (tag, name)
    cfg = dict(dtype="mxfp4", scale_rule="static_6")
    for mm in gold["matmuls"]:
        qa, qb = oracle.quantize(gold["inputs"][mm["a"]], **cfg), oracle.quantize(gold["inputs"][mm["b"]], **cfg)
        assert oracle.alpha(qa, qb) == 1.0
        dt = getattr(torch, mm["out_dtype"])
        out = oracle.matmul(qa, qb, dt)
        if dt == torch.float32:
            denom = mm["out"].abs().max().clamp_min(1e-30)
            assert ((out - mm["out"]).abs().max() / denom).item() < 1e-5
        else:
            assert (out != mm["out"]).float().mean().item() <= 1e-3
