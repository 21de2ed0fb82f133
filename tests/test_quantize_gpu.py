"""Parity of the CUDA quantize / dequantize kernels with the reference, on a B200.

Three layers, all bit-exact (codes, scales, amax, hence every 4-vs-6 / int-vs-float
block choice):
  1. the committed golden vectors produced by the reference's PyTorch backend,
  2. the CPU oracle on larger seeded inputs, following the parameter sweep of the
     reference's tests/test_quantize.py:23-314 (input kinds, shapes, rules, 2-D blocks,
     transposition, formats, several seeds),
  3. the benchmark's full-size tensors against the oracle.
Every comparison also asserts that no scaled magnitude reached 7, the point where the
reference's unclamped rounding and the hardware's saturating conversion would part ways.
"""

from __future__ import annotations

import pytest
import torch

import fouroversix_b200 as fos
from fouroversix_b200.quantize.backend import B200QuantizeBackend

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _cfg(d: dict) -> fos.QuantizationConfig:
    return fos.QuantizationConfig(**{k: v for k, v in d.items() if k != "backend"})


def _assert_same(q: fos.QuantizedTensor, values, scales, amax, name):
    torch.cuda.synchronize()
    got_v, got_s = q.values.cpu(), q.scale_factors.view(torch.uint8).flatten().cpu()
    n_v, n_s = int((got_v != values).sum()), int((got_s != scales).sum())
    assert n_v == 0 and n_s == 0, f"{name}: {n_v} code bytes and {n_s} scale bytes differ"
    assert torch.equal(q.amax.cpu().reshape(1), amax.reshape(1)), name


@pytest.mark.parametrize("exact_only", [False, True], ids=["fast-filter", "exact-only"])
def test_golden_vectors(golden, exact_only):
    for case in golden["cases"]:
        x = golden["inputs"][case["input"]].to(DEV)
        cfg = _cfg(case["config"])
        q = B200QuantizeBackend.quantize(x, cfg, exact_only=exact_only)
        assert q.padded_shape == tuple(case["padded_shape"]) and q.original_shape == tuple(case["original_shape"])
        assert q.scale_factors_are_in_blackwell_layout == case["tiled"]
        _assert_same(q, case["values"], case["scale_factors"], case["amax"], case["name"])
        for key, dt in (("dequant_bf16", torch.bfloat16), ("dequant_fp16", torch.float16),
                        ("dequant_fp32", torch.float32)):
            if key in case:
                out = fos.dequantize(q, dt).cpu()
                view = torch.int32 if dt == torch.float32 else torch.int16
                assert torch.equal(out.view(view), case[key].contiguous().view(view)), (case["name"], key)


def _make_input(kind: str, shape, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    if kind == "zeros":
        return torch.zeros(shape, dtype=torch.bfloat16)
    if kind == "ones":
        return torch.ones(shape, dtype=torch.bfloat16)
    if kind == "rand01":
        return torch.rand(shape, generator=g).bfloat16()
    if kind == "outlier":
        a = torch.randn(shape, generator=g)
        a[:, torch.randperm(shape[1], generator=g)[: max(1, shape[1] // 100)]] *= 20
        return a.bfloat16()
    if kind == "small":
        return (torch.randn(shape, generator=g) * 0.02).bfloat16()
    return torch.randn(shape, generator=g).bfloat16()


SWEEP_RULES = {"nvfp4": ["abs_max", "mae", "mse", "static_4", "static_6"], "if4": ["abs_max", "mae", "mse"]}


@pytest.mark.parametrize("kind", ["zeros", "ones", "rand01", "randn", "outlier", "small"])
@pytest.mark.parametrize("shape", [(1024, 1024), (1024, 512), (512, 1024)])
def test_sweep_against_oracle(oracle, kind, shape):
    seeds = [0] if kind in ("zeros", "ones") else [0, 1, 2]
    for seed in seeds:
        x = _make_input(kind, shape, seed)
        xd = x.to(DEV)
        for dtype, rules in SWEEP_RULES.items():
            for rule in rules:
                for two_d in (False, True):
                    for transpose in (False, True):
                        cfg = fos.QuantizationConfig(dtype=dtype, scale_rule=rule, block_scale_2d=two_d,
                                                     transpose=transpose)
                        q = fos.quantize(xd, cfg)
                        ref = oracle.quantize(x, dtype=dtype, scale_rule=rule, block_scale_2d=two_d,
                                              transpose=transpose)
                        assert ref.worst_scaled < 7.0
                        name = f"{kind}{shape} seed{seed} {dtype} {rule} 2d={two_d} t={transpose}"
                        _assert_same(q, ref.values, ref.scale_factors, ref.amax, name)


def test_dequantize_against_oracle(oracle):
    x = _make_input("randn", (384, 320), 5)
    for dtype, rule in [("nvfp4", "mse"), ("nvfp4", "static_6"), ("nvfp4", "static_4"), ("if4", "mse")]:
        q = fos.quantize(x.to(DEV), fos.QuantizationConfig(dtype=dtype, scale_rule=rule))
        ref = oracle.quantize(x, dtype=dtype, scale_rule=rule)
        for out_dtype, view in [(torch.bfloat16, torch.int16), (torch.float16, torch.int16),
                                (torch.float32, torch.int32)]:
            got = fos.dequantize(q, out_dtype).cpu()
            want = oracle.dequantize(ref, out_dtype)
            assert torch.equal(got.view(view), want.view(view)), (dtype, rule, out_dtype)
        # fused fake-quantization = quantize then dequantize in the input's dtype
        fake = fos.quantize(x.to(DEV), fos.QuantizationConfig(dtype=dtype, scale_rule=rule, pseudo_quantize=True))
        assert torch.equal(fake.cpu().view(torch.int16), oracle.dequantize(ref, torch.bfloat16).view(torch.int16))


def test_ragged_unaligned_strided_and_fp16_inputs(oracle):
    g = torch.Generator().manual_seed(11)
    wide = torch.randn(256, 512, generator=g).bfloat16()
    wide_dev = wide.to(DEV)
    cases = [  # (CPU tensor, the same tensor on the GPU)
        (a, a.to(DEV)) for a in (
            torch.randn(100, 80, generator=g).bfloat16(),
            torch.randn(37, 53, generator=g).bfloat16(),        # nothing aligned, partial blocks
            torch.randn(130, 200, generator=g).half(),
        )
    ] + [
        (wide[:, 8:264], wide_dev[:, 8:264]),                    # row stride != width, 16-byte aligned only
        (wide[:, 3:200], wide_dev[:, 3:200]),                    # unaligned start, ragged width
        (wide[5:200, 16:80], wide_dev[5:200, 16:80]),
    ]
    for x, xd in cases:
        assert xd.stride() == x.stride()
        for cfg in (dict(), dict(scale_rule="static_6"), dict(dtype="if4"), dict(block_scale_2d=True)):
            q = fos.quantize(xd, fos.QuantizationConfig(**cfg))
            ref = oracle.quantize(x, **cfg)
            _assert_same(q, ref.values, ref.scale_factors, ref.amax, f"{tuple(x.shape)} {x.dtype} {cfg}")
            got = fos.dequantize(q).cpu()
            assert got.shape == x.shape
            assert torch.equal(got.view(torch.int16), oracle.dequantize(ref).view(torch.int16))


def test_caller_supplied_amax_skips_the_reduction(oracle):
    x = _make_input("randn", (256, 256), 3)
    xd = x.to(DEV)
    amax = xd.abs().max().float().reshape(1)
    q = B200QuantizeBackend.quantize(xd, fos.QuantizationConfig(), amax=amax)
    ref = oracle.quantize(x)
    _assert_same(q, ref.values, ref.scale_factors, ref.amax, "amax given")


@pytest.mark.parametrize("name,shape,seed,cfg", [
    ("c1-4096x4096-mse", (4096, 4096), 0, dict()),
    ("c1-4096x4096-static6", (4096, 4096), 0, dict(scale_rule="static_6")),
    ("c2-act-8192x4096-mse", (8192, 4096), 1, dict()),
    ("c3-if4-4096x4096", (4096, 4096), 5, dict(dtype="if4")),
    ("c4-weight-2d", (4096, 4096), 10, dict(block_scale_2d=True)),
    ("c4-act-transposed", (4096, 4096), 9, dict(transpose=True)),
])
def test_full_size_configs_bit_exact(oracle, name, shape, seed, cfg):
    kind = "outlier" if name.startswith("c2") else ("small" if "weight" in name else "randn")
    x = _make_input(kind, shape, seed)
    q = fos.quantize(x.to(DEV), fos.QuantizationConfig(**cfg))
    ref = oracle.quantize(x, **cfg)
    assert ref.worst_scaled < 7.0
    _assert_same(q, ref.values, ref.scale_factors, ref.amax, name)
    # round trip: dequantize(quantize(x)) stays within half an FP4 step of x everywhere
    back = fos.dequantize(q, torch.float32).cpu()
    xf = x.float().T if cfg.get("transpose") else x.float()
    assert (back - xf).abs().max() <= 0.26 * x.float().abs().max()


@pytest.mark.parametrize("kernel", ["auto", "general", "no_tma"], ids=["specialised", "tma-fed", "register-loads"])
def test_both_row_kernels_match_the_oracle(oracle, kernel):
    """1-D untransposed inputs have three kernels (the one for NVFP4 4/6 MSE alone, the general one fed by
    the TMA unit, the one loading into registers; a per-call flag picks one);
    all must give the reference's bytes, with and without a caller-supplied amax (the first
    walks the tiles forwards, the second backwards), on full, ragged and tiny shapes."""
    import ctypes

    from fouroversix_b200 import _native

    lib = _native.lib()
    g = torch.Generator().manual_seed(21)
    shapes = [(8, 16), (100, 80), (129, 72), (128, 64), (640, 4096), (1000, 328), (257, 8200)]
    try:
        for shape in shapes:
            x = torch.randn(shape, generator=g).bfloat16()
            x[:, :: 7] *= 9.0
            xd = x.to(DEV)
            amax = xd.abs().max().float().reshape(1)
            for cfg in (dict(), dict(scale_rule="static_6"), dict(scale_rule="static_4"), dict(scale_rule="mae"),
                        dict(scale_rule="abs_max"), dict(dtype="if4"), dict(block_scale_2d=True),
                        dict(block_scale_2d=True, scale_rule="static_6"), dict(block_scale_2d=True, dtype="if4")):
                ref = oracle.quantize(x, **cfg)
                for given in (None, amax):
                    q = B200QuantizeBackend.quantize(xd, fos.QuantizationConfig(**cfg), amax=given, kernel=kernel)
                    _assert_same(q, ref.values, ref.scale_factors, ref.amax, f"{shape} {cfg} amax given={given is not None}")
        # transposed inputs have the same pair of kernels (sizes the reference accepts: multiples of 128)
        for shape in [(128, 256), (640, 4096), (1152, 384)]:
            x = torch.randn(shape, generator=g).bfloat16()
            x[:: 5, :] *= 7.0
            xd = x.to(DEV)
            amax = xd.abs().max().float().reshape(1)
            for cfg in (dict(transpose=True), dict(transpose=True, scale_rule="static_6"), dict(transpose=True, dtype="if4"),
                        dict(transpose=True, scale_rule="abs_max"), dict(transpose=True, block_scale_2d=True),
                        dict(transpose=True, block_scale_2d=True, scale_rule="mae")):
                ref = oracle.quantize(x, **cfg)
                for given in (None, amax):
                    q = B200QuantizeBackend.quantize(xd, fos.QuantizationConfig(**cfg), amax=given, kernel=kernel)
                    _assert_same(q, ref.values, ref.scale_factors, ref.amax, f"{shape} {cfg} amax given={given is not None}")
        xh = torch.randn(300, 264, generator=g).half()
        ref = oracle.quantize(xh)
        q = B200QuantizeBackend.quantize(xh.to(DEV), fos.QuantizationConfig(), kernel=kernel)
        _assert_same(q, ref.values, ref.scale_factors, ref.amax, "fp16 300x264")
    finally:
        pass
    site = ctypes.c_int32(-1)
    assert lib.fos_wait_failure_site(ctypes.byref(site)) == 0 and site.value == 0


def test_fused_fake_quantization_equals_quantize_then_dequantize(oracle):
    """pseudo_quantize: the fused kernel (aligned inputs) and the two-kernel path (anything else) give
    the bits of the oracle's quantize followed by its dequantize, in the input's dtype, on full,
    ragged and strided inputs."""
    g = torch.Generator().manual_seed(31)
    wide = torch.randn(300, 520, generator=g).bfloat16()
    wide_dev = wide.to(DEV)
    cases = [(a, a.to(DEV)) for a in (
        torch.randn(256, 512, generator=g).bfloat16(),
        torch.randn(100, 80, generator=g).bfloat16(),
        torch.randn(37, 53, generator=g).bfloat16(),            # unaligned rows: two-kernel path
        torch.randn(130, 200, generator=g).half(),
        (torch.randn(1024, 4096, generator=g) * 0.02).bfloat16(),
    )] + [(wide[:, 8:264], wide_dev[:, 8:264]), (wide[3:200, 16:500], wide_dev[3:200, 16:500])]
    for x, xd in cases:
        for cfg in (dict(), dict(scale_rule="static_6"), dict(dtype="if4"), dict(scale_rule="mae")):
            ref = oracle.quantize(x, **cfg)
            want = oracle.dequantize(ref, x.dtype)
            got = fos.quantize(xd, fos.QuantizationConfig(pseudo_quantize=True, **cfg))
            assert got.dtype == x.dtype and got.shape == x.shape
            assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16)), (tuple(x.shape), x.dtype, cfg)


@pytest.mark.parametrize("kernel", ["auto", "no_tma"], ids=["tma-fed", "register-loads"])
def test_random_hadamard_transform_matches_reference_and_oracle(oracle, kernel):
    """QuantizationConfig.rht: the committed vectors of the reference (rotation + quantization on
    CPU) and larger seeded inputs against the oracle, plain and transposed, with both kernel families."""
    import io
    import lzma
    from pathlib import Path

    from fouroversix_b200 import _native

    raw = lzma.decompress((Path(__file__).parent / "golden" / "reference_golden_rht.pt.xz").read_bytes())
    gold = torch.load(io.BytesIO(raw), weights_only=False)
    try:
        for case in gold["cases"]:
            x = gold["inputs"][case["input"]]
            q = B200QuantizeBackend.quantize(x.to(DEV), fos.QuantizationConfig(rht=True, **case["config"]), kernel=kernel)
            torch.cuda.synchronize()
            v = case["values"]
            assert torch.equal(q.values.cpu()[: v.shape[0], : v.shape[1]], v), (case["input"], case["config"])
            n = case["scale_factors"].numel()
            assert torch.equal(q.scale_factors.view(torch.uint8).flatten().cpu()[:n], case["scale_factors"])
            assert torch.equal(q.amax.cpu().reshape(1), case["amax"])
        g = torch.Generator().manual_seed(41)
        for shape in [(1024, 512), (640, 4096), (384, 1152)]:
            x = (torch.randn(shape, generator=g) * 3e-3).bfloat16()
            xd = x.to(DEV)
            for cfg in (dict(), dict(transpose=True), dict(transpose=True, scale_rule="static_6"), dict(dtype="if4"),
                        dict(transpose=True, block_scale_2d=True)):
                ref = oracle.quantize(x, rht=True, **cfg)
                q = B200QuantizeBackend.quantize(xd, fos.QuantizationConfig(rht=True, **cfg), kernel=kernel)
                _assert_same(q, ref.values, ref.scale_factors, ref.amax, f"rht {shape} {cfg}")
    finally:
        pass


def test_stochastic_rounding_statistics():
    """RoundStyle.stochastic. The reference's generator cannot be reproduced, so the checks are the
    ones its own test makes (tests/test_quantize.py:317-388: distance between x and its quantized
    copy on a 1024 x 1024 N(0,1) tensor, 137 for static_6 and 122 for the 4/6 MSE rule with its
    Triton kernels, 141 with TransformerEngine, each +-5 %) plus what defines the method: every value
    lands on one of the two grid points around it, the mean over many seeds approaches x, the same
    seed repeats and another seed does not."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1024, 1024, generator=g).bfloat16()
    xd = x.to(DEV)
    for rule, lo, hi in (("static_6", 137 * 0.95, 141 * 1.05), ("mse", 122 * 0.95, 126 * 1.05)):
        cfg = fos.QuantizationConfig(scale_rule=rule, round_style="stochastic")
        q1 = B200QuantizeBackend.quantize(xd, cfg, seed=11)
        q2 = B200QuantizeBackend.quantize(xd, cfg, seed=11)
        q3 = B200QuantizeBackend.quantize(xd, cfg, seed=12)
        assert torch.equal(q1.values, q2.values) and torch.equal(q1.scale_factors.view(torch.uint8), q2.scale_factors.view(torch.uint8))
        assert not torch.equal(q1.values, q3.values)
        dist = torch.dist(fos.dequantize(q1, torch.float32), xd.float()).item()
        assert lo <= dist <= hi, (rule, dist)
    # static_6: same scales as round-to-nearest, every code within one grid step of the nearest one,
    # and the average over seeds converges to x (round-to-nearest has a fixed error instead)
    cfg = fos.QuantizationConfig(scale_rule="static_6", round_style="stochastic")
    near = fos.quantize(xd, fos.QuantizationConfig(scale_rule="static_6"))
    acc = torch.zeros_like(xd, dtype=torch.float32)
    n_seeds = 64
    for seed in range(n_seeds):
        q = B200QuantizeBackend.quantize(xd, cfg, seed=seed)
        assert torch.equal(q.scale_factors.view(torch.uint8), near.scale_factors.view(torch.uint8))
        acc += fos.dequantize(q, torch.float32)
    mean_err = (acc / n_seeds - xd.float()).pow(2).mean().sqrt().item()
    near_err = (fos.dequantize(near, torch.float32) - xd.float()).pow(2).mean().sqrt().item()
    assert mean_err < 0.35 * near_err, (mean_err, near_err)
    # transposed + rotated (the wgrad configuration) runs and repeats
    cfg = fos.QuantizationConfig(round_style="stochastic", transpose=True, rht=True)
    qa = B200QuantizeBackend.quantize(xd, cfg, seed=5)
    qb = B200QuantizeBackend.quantize(xd, cfg, seed=5)
    assert torch.equal(qa.values, qb.values) and qa.padded_shape == (1024, 1024)


def test_stochastic_unbiased_rounding():
    """RoundStyle.stochastic_unbiased (src/fouroversix/utils.py:223-247): stochastic rounding with every maximum
    scaled by 16/17. Scale bytes are deterministic for a static rule and must equal the reference's formula
    (src/fouroversix/quantize/pytorch/reference.py:203-218, checked against the reference's own scale bytes where
    it can be imported); the distances are the reference's pinned ones (tests/test_quantize.py:318-362: 158 for
    static_6, 139 for 4/6 MSE, +-5 %); the mean over seeds approaches x; dequantize and the GEMM's alpha carry
    the same factor."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1024, 1024, generator=g).bfloat16()
    xd = x.to(DEV)
    amax = x.float().abs().max()
    encode = torch.tensor(6 * 448 * (16 / 17), dtype=torch.float32) / amax
    hp = x.float().reshape(1024, 64, 16).abs().amax(-1) / torch.tensor(6 * (16 / 17), dtype=torch.float32) * encode
    want_sf = hp.to(torch.float8_e4m3fn).view(torch.uint8)
    cfg = fos.QuantizationConfig(scale_rule="static_6", round_style="stochastic_unbiased")
    q = B200QuantizeBackend.quantize(xd, cfg, seed=3)
    assert q.round_style is fos.RoundStyle.stochastic_unbiased
    from fouroversix_b200.quantize import from_blocked

    assert torch.equal(from_blocked(q.scale_factors.cpu(), (1024, 64)).view(torch.uint8), want_sf)
    for rule, pinned in (("static_6", 158.0), ("mse", 139.0)):
        c = fos.QuantizationConfig(scale_rule=rule, round_style="stochastic_unbiased")
        q1, q2 = B200QuantizeBackend.quantize(xd, c, seed=11), B200QuantizeBackend.quantize(xd, c, seed=11)
        assert torch.equal(q1.values, q2.values)
        dist = torch.dist(fos.dequantize(q1, torch.float32), xd.float()).item()
        assert pinned * 0.95 <= dist <= pinned * 1.05, (rule, dist)
    acc = torch.zeros_like(xd, dtype=torch.float32)
    for seed in range(64):
        acc += fos.dequantize(B200QuantizeBackend.quantize(xd, cfg, seed=seed), torch.float32)
    near = fos.quantize(xd, fos.QuantizationConfig(scale_rule="static_6"))
    mean_err = (acc / 64 - xd.float()).pow(2).mean().sqrt().item()
    near_err = (fos.dequantize(near, torch.float32) - xd.float()).pow(2).mean().sqrt().item()
    assert mean_err < 0.35 * near_err, (mean_err, near_err)
    # the factor in dequantize: the same packed bytes read as a plain stochastic tensor are 16/17 times as large
    plain = fos.QuantizedTensor(q.values, q.scale_factors, q.amax, q.dtype, q.original_shape, q.scale_rule, "stochastic",
                                q.padded_shape, scale_factors_are_in_blackwell_layout=True)
    a, b = fos.dequantize(q, torch.float32), fos.dequantize(plain, torch.float32)
    assert torch.allclose(a * (16 / 17), b, rtol=1e-6, atol=0)
    # and in the GEMM's alpha
    w = fos.quantize((torch.randn(256, 1024, generator=g) * 0.05).bfloat16().to(DEV))
    ya = fos.quantized_matmul(q, w, out_dtype=fos.DataType.float32)
    yb = fos.quantized_matmul(plain, w, out_dtype=fos.DataType.float32)
    assert torch.allclose(ya * (16 / 17), yb, rtol=1e-5, atol=0)


def test_stochastic_rounding_if4():
    """IF4 with stochastic rounding: both grids draw independent noise and the smaller squared error of the draw
    wins. Parity in distribution, by the reference's pinned distances (tests/test_quantize.py:322: 110, and 122 for
    stochastic_unbiased, +-5 %); the mean over seeds approaches x; same seed, same bytes; both grids are in use."""
    g = torch.Generator().manual_seed(0)
    xd = torch.randn(1024, 1024, generator=g).bfloat16().to(DEV)
    for style, pinned in (("stochastic", 110.0), ("stochastic_unbiased", 122.0)):
        c = fos.QuantizationConfig(dtype="if4", scale_rule="mse", round_style=style)
        q1, q2 = B200QuantizeBackend.quantize(xd, c, seed=5), B200QuantizeBackend.quantize(xd, c, seed=5)
        q3 = B200QuantizeBackend.quantize(xd, c, seed=6)
        assert torch.equal(q1.values, q2.values) and torch.equal(q1.scale_factors.view(torch.uint8), q2.scale_factors.view(torch.uint8))
        assert not torch.equal(q1.values, q3.values)
        dist = torch.dist(fos.dequantize(q1, torch.float32), xd.float()).item()
        assert pinned * 0.95 <= dist <= pinned * 1.05, (style, dist)
        int_blocks = (q1.scale_factors.view(torch.uint8) >= 128).float().mean().item()
        assert 0.05 < int_blocks < 0.95, int_blocks
    c = fos.QuantizationConfig(dtype="if4", scale_rule="mse", round_style="stochastic")
    acc = torch.zeros_like(xd, dtype=torch.float32)
    for seed in range(64):
        acc += fos.dequantize(B200QuantizeBackend.quantize(xd, c, seed=seed), torch.float32)
    near = fos.quantize(xd, fos.QuantizationConfig(dtype="if4", scale_rule="mse"))
    mean_err = (acc / 64 - xd.float()).pow(2).mean().sqrt().item()
    near_err = (fos.dequantize(near, torch.float32) - xd.float()).pow(2).mean().sqrt().item()
    assert mean_err < 0.5 * near_err, (mean_err, near_err)
    with pytest.raises(ValueError):
        fos.quantize(xd, fos.QuantizationConfig(dtype="if4", scale_rule="mae", round_style="stochastic"))


def _load_golden_file(name: str):
    import io
    import lzma
    from pathlib import Path

    raw = lzma.decompress((Path(__file__).parent / "golden" / name).read_bytes())
    return torch.load(io.BytesIO(raw), weights_only=False)


def test_mxfp4_matches_reference_and_oracle(oracle):
    """MXFP4 (E8M0 scale per 32 values; static_6 / static_4; 1-D and 32 x 32 blocks; transposed):
    the reference's own outputs (golden file: codes, scales, dequantized bits in three types), then
    the oracle on larger, ragged, strided and fp16 inputs."""
    gold = _load_golden_file("reference_golden_mxfp4.pt.xz")
    for case in gold["cases"]:
        tag = (case["input"], case["config"])
        x = gold["inputs"][case["input"]].to(DEV)
        q = fos.quantize(x, fos.QuantizationConfig(dtype="mxfp4", **case["config"]))
        assert q.padded_shape == case["padded_shape"] and q.original_shape == case["original_shape"], tag
        assert q.scale_factors.dtype == torch.float8_e8m0fnu and q.scale_factors_are_in_blackwell_layout
        _assert_same(q, case["values"], case["scale_factors"], case["amax"], tag)
        for name, ref in case["dequantized"].items():
            dt = getattr(torch, name)
            out = fos.dequantize(q, dt).cpu()
            view = torch.int32 if dt == torch.float32 else torch.int16
            # 0 x inf (a block scale beyond fp16's range) is NaN on both sides; its payload is the platform's
            nan = torch.isnan(ref)
            assert torch.equal(torch.isnan(out), nan), (tag, name)
            assert torch.equal(out.view(view)[~nan], ref.contiguous().view(view)[~nan]), (tag, name)
    g = torch.Generator().manual_seed(77)
    big = torch.randn(1024, 2048, generator=g)
    big[:, torch.randperm(2048, generator=g)[:20]] *= 20.0
    inputs = {
        "outliers_1024x2048": big.bfloat16(),
        "weights_384x640": (torch.randn(384, 640, generator=g) * 0.02).bfloat16(),
        "ragged_333x217": torch.randn(333, 217, generator=g).bfloat16(),
        "half_200x96": torch.randn(200, 96, generator=g).half(),
        "odd_129x33": (torch.randn(129, 33, generator=g) * 1e-3).bfloat16(),
    }
    for name, x in inputs.items():
        for kw in (dict(scale_rule="static_6"), dict(scale_rule="static_4"), dict(scale_rule="static_6", transpose=True),
                   dict(scale_rule="static_6", block_scale_2d=True), dict(scale_rule="static_4", block_scale_2d=True, transpose=True)):
            ref = oracle.quantize(x, dtype="mxfp4", **kw)
            q = fos.quantize(x.to(DEV), fos.QuantizationConfig(dtype="mxfp4", **kw))
            assert q.padded_shape == ref.padded_shape and q.original_shape == ref.original_shape
            _assert_same(q, ref.values, ref.scale_factors, ref.amax, (name, kw))
            out = fos.dequantize(q, torch.bfloat16).cpu()
            assert torch.equal(out.view(torch.int16), oracle.dequantize(ref, torch.bfloat16).view(torch.int16)), (name, kw)
    # a view with a row stride (every other row of a wider tensor; 16-byte alignment lost)
    wide = torch.randn(256, 300, generator=g).bfloat16()
    view = wide.to(DEV)[::2, 3:259]
    ref = oracle.quantize(wide[::2, 3:259].contiguous(), dtype="mxfp4", scale_rule="static_6")
    q = fos.quantize(view, fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6"))
    _assert_same(q, ref.values, ref.scale_factors, ref.amax, "strided view")
    # what the format does not define is refused
    with pytest.raises(ValueError):
        fos.quantize(view, fos.QuantizationConfig(dtype="mxfp4", scale_rule="mse"))
    # fake quantization = quantize then dequantize
    x = inputs["weights_384x640"].to(DEV)
    cfg = fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6")
    fake = fos.quantize(x, fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6", pseudo_quantize=True))
    assert torch.equal(fake.view(torch.int16), fos.dequantize(fos.quantize(x, cfg), torch.bfloat16).view(torch.int16))


def test_float32_intermediate_and_raw_values_match_the_reference():
    """`dequantize(..., intermediate_dtype=torch.float32)` (what the reference's own pseudo-quantize test uses,
    tests/test_quantize.py:442) and `dequantize_values`, bit for bit against outputs of the reference's PyTorch
    backend on tensors it quantized itself (tests/golden/make_golden_dequant32.py)."""
    import io
    import lzma
    from pathlib import Path

    raw = lzma.decompress((Path(__file__).parent / "golden" / "reference_golden_dequant32.pt.xz").read_bytes())
    gold = torch.load(io.BytesIO(raw), weights_only=False)
    assert len(gold["cases"]) == 20
    for case in gold["cases"]:
        cfg = case["config"]
        scale_dtype = torch.float8_e8m0fnu if cfg["dtype"] == "mxfp4" else torch.float8_e4m3fn
        q = fos.QuantizedTensor(case["values"].to(DEV), case["scale_factors"].to(DEV).view(scale_dtype),
                                None if case["amax"] is None else case["amax"].to(DEV), cfg["dtype"], case["original_shape"],
                                case["scale_rule"], "nearest", case["padded_shape"],
                                scale_factors_are_in_blackwell_layout=case["tiled"])
        what = (case["input"], cfg)
        for dtype, key in ((torch.bfloat16, "dequant32_bf16"), (torch.float32, "dequant32_fp32")):
            got = fos.dequantize(q, dtype, intermediate_dtype=torch.float32)
            want = case[key]
            assert got.shape == want.shape and got.dtype == want.dtype, what
            assert torch.equal(got.cpu().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                               want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32)), (what, key)
        for dtype, key in ((torch.float16, "values_fp16"), (torch.float32, "values_fp32")):
            got = B200QuantizeBackend.dequantize_values(q, dtype=dtype)
            want = case[key]
            assert got.shape == want.shape, what
            assert torch.equal(got.cpu().view(torch.int16 if dtype == torch.float16 else torch.int32),
                               want.view(torch.int16 if dtype == torch.float16 else torch.int32)), (what, key)
    with pytest.raises(ValueError, match="intermediate"):
        fos.dequantize(q, torch.bfloat16, intermediate_dtype=torch.bfloat16)
