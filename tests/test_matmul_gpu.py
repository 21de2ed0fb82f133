"""Parity of the tcgen05 block-scaled FP4 GEMM with the reference's matmul semantics.

Operands are quantized once and fed to both sides, as in the reference's
tests/test_matmul.py:19-88.  The other side is the oracle: bf16(deq32(a) @ deq32(b).T).
Criteria: at most 0.1 % of bf16 outputs differ (the reference's own cross-backend bar,
tests/test_matmul.py:15) and max |error| <= 1e-2 * max |reference| against the fp32
product of the dequantized operands.
"""

from __future__ import annotations

import itertools

import pytest
import torch

import fouroversix_b200 as fos
from fouroversix_b200 import _native
from fouroversix_b200.matmul import B200MatmulBackend

pytestmark = pytest.mark.gpu

DEV = "cuda"
MISMATCH_TOLERANCE = 1e-3
REL_TOLERANCE = 1e-2


def _dense_reference(qa: fos.QuantizedTensor, qb: fos.QuantizedTensor) -> torch.Tensor:
    """fp32 product of the dequantized operands, on the GPU with TF32 off (the dequantize
    kernel itself is checked bit for bit against the oracle elsewhere)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return fos.dequantize(qa, torch.float32) @ fos.dequantize(qb, torch.float32).T
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def _check(out: torch.Tensor, ref32: torch.Tensor, what: str, mismatch_scale: float = 1.0):
    torch.cuda.synchronize()
    assert out.shape == ref32.shape, what
    assert torch.isfinite(out.float()).all(), what
    denom = ref32.abs().max().clamp_min(1e-30)
    rel = ((out.float() - ref32).abs().max() / denom).item()
    assert rel <= REL_TOLERANCE, f"{what}: max relative error {rel}"
    frac = (out != ref32.to(out.dtype)).float().mean().item()
    # the 0.1 % bar is the reference's for bf16 outputs; fp16 keeps 3 more mantissa bits, so the
    # same fp32 summation-order noise flips 8 times as many roundings
    # ... and both sides accumulate K products in fp32 in different orders; that noise grows like
    # sqrt(K), so beyond the reference test's largest K (1024) the bar grows by sqrt(K / 1024)
    tol = MISMATCH_TOLERANCE * (8 if out.dtype == torch.float16 else 1) * mismatch_scale
    assert frac <= tol, f"{what}: {frac:.3%} of outputs differ"


def _synthetic(rows: int, k: int, code_byte: int, scale_byte: int) -> fos.QuantizedTensor:
    """A quantized tensor built by hand: every code byte and scale byte the same, amax chosen
    so that alpha = 1 for static_6 operands."""
    values = torch.full((rows, k // 2), code_byte, dtype=torch.uint8, device=DEV)
    scales = torch.full((rows * k // 16,), scale_byte, dtype=torch.uint8, device=DEV).view(torch.float8_e4m3fn)
    amax = torch.full((1,), 2688.0, dtype=torch.float32, device=DEV)
    return fos.QuantizedTensor(values, scales, amax, "nvfp4", (rows, k), "static_6", "nearest", (rows, k))


@pytest.mark.parametrize("block_n", [128, 256, 2])
def test_hand_built_operands(block_n):
    """All ones times all ones is K; then random codes and scales catch a wrong scale-tile or
    swizzle mapping. `block_n` selects the kernel: single-CTA 128- or 256-wide tiles, or 2 =
    the CTA-pair kernel."""
    try:
        m, n, k = 256, 256, 512
        a, b = _synthetic(m, k, 0x22, 0x38), _synthetic(n, k, 0x22, 0x38)     # 1.0 values, 1.0 scales
        out = B200MatmulBackend.quantized_matmul(a, b, out_dtype=fos.DataType.float32, check_status=True, variant=block_n)
        assert torch.equal(out, torch.full((m, n), float(k), device=DEV))

        g = torch.Generator().manual_seed(0)
        a.values.copy_(torch.randint(0, 256, a.values.shape, generator=g, dtype=torch.uint8))
        b.values.copy_(torch.randint(0, 256, b.values.shape, generator=g, dtype=torch.uint8))
        # positive, finite E4M3 scales between 2^-3 and 8
        a.scale_factors.view(torch.uint8).copy_(torch.randint(0x20, 0x50, (m * k // 16,), generator=g, dtype=torch.uint8))
        b.scale_factors.view(torch.uint8).copy_(torch.randint(0x20, 0x50, (n * k // 16,), generator=g, dtype=torch.uint8))
        out = B200MatmulBackend.quantized_matmul(a, b, out_dtype=fos.DataType.float32, check_status=True, variant=block_n)
        ref = _dense_reference(a, b)
        # every product is exactly representable and the sums stay below 2^24 ulps: tight bound
        assert ((out - ref).abs().max() / ref.abs().max()).item() < 1e-5
    finally:
        pass


@pytest.mark.parametrize(("m", "n", "k"), list(itertools.product([256, 512, 1024], repeat=3)))
@pytest.mark.parametrize("scale_rule", ["static_6", "static_4", "mse"])
@pytest.mark.parametrize("variant", [0, 2], ids=["auto", "cta-pair"])
def test_matmul_against_oracle(oracle, m, n, k, scale_rule, variant):
    _matmul_against_oracle(oracle, m, n, k, scale_rule, variant)


def _matmul_against_oracle(oracle, m, n, k, scale_rule, variant=0):
    for seed in range(2):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(m, k, generator=g).bfloat16()
        y = torch.randn(n, k, generator=g).bfloat16()
        cfg = fos.QuantizationConfig(scale_rule=scale_rule)
        qx, qy = fos.quantize(x.to(DEV), cfg), fos.quantize(y.to(DEV), cfg)
        out = B200MatmulBackend.quantized_matmul(qx, qy, out_dtype=fos.DataType.bfloat16, check_status=True, variant=variant)
        ox, oy = oracle.quantize(x, scale_rule=scale_rule), oracle.quantize(y, scale_rule=scale_rule)
        want = oracle.matmul(ox, oy, torch.bfloat16) if m * n * k <= 256 * 512 * 1024 else None
        ref32 = _dense_reference(qx, qy)
        _check(out, ref32, f"{m}x{n}x{k} {scale_rule} seed {seed}")
        if want is not None:
            frac = (out.cpu() != want).float().mean().item()
            assert frac <= MISMATCH_TOLERANCE, f"vs oracle matmul: {frac:.3%} differ"


def test_golden_matmul_cases(golden):
    for mm in golden["matmul"]:
        ca, cb = mm["cfg_a"], mm["cfg_b"]
        out = fos.quantized_matmul(mm["a"].to(DEV), mm["b"].to(DEV), input_config=fos.QuantizationConfig(**ca),
                                   other_config=fos.QuantizationConfig(**cb), check_status=True)
        want = mm["out_bf16"]
        assert out.shape == want.shape
        frac = (out.cpu() != want).float().mean().item()
        assert frac <= MISMATCH_TOLERANCE, (ca, cb, frac)
        rel = ((out.cpu().float() - mm["out_fp32"]).abs().max() / mm["out_fp32"].abs().max()).item()
        assert rel <= REL_TOLERANCE


@pytest.mark.parametrize("shape", [(100, 72, 80), (130, 300, 192), (128, 128, 64), (257, 129, 1000), (384, 640, 448),
                                   (512, 768, 448), (256, 256, 64), (500, 1000, 320)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float16", "float32"])
def test_ragged_shapes_and_output_types(shape, out_dtype):
    m, n, k = shape
    g = torch.Generator().manual_seed(7)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    y = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(DEV)
    qx, qy = fos.quantize(x), fos.quantize(y)
    for block_n in (128, 256, 2):
        out = B200MatmulBackend.quantized_matmul(qx, qy, out_dtype=fos.DataType(out_dtype), check_status=True, variant=block_n)
        ref32 = _dense_reference(qx, qy)
        if out_dtype == "float32":
            assert ((out - ref32).abs().max() / ref32.abs().max()).item() < 1e-5
        else:
            _check(out, ref32, f"{shape} {out_dtype} block_n={block_n}")


def test_output_is_cropped_and_nothing_else_is_written():
    m, n, k = 100, 72, 128
    g = torch.Generator().manual_seed(3)
    qx = fos.quantize(torch.randn(m, k, generator=g).bfloat16().to(DEV))
    qy = fos.quantize(torch.randn(n, k, generator=g).bfloat16().to(DEV))
    canvas = torch.full((m + 2, n + 8), 7.0, dtype=torch.bfloat16, device=DEV)
    view = canvas[1:m + 1, :n]
    B200MatmulBackend.quantized_matmul(qx, qy, out_dtype=fos.DataType.bfloat16, out=view, check_status=True)
    torch.cuda.synchronize()
    assert (canvas[0] == 7).all() and (canvas[-1] == 7).all() and (canvas[:, n:] == 7).all()
    _check(view, _dense_reference(qx, qy), "cropped")


def test_skinny_problem_bound_by_memory():
    """One row block against a weight far larger than L2, K not a multiple of the stage: every CTA streams
    its B tiles from HBM and the loads of a stage land out of order. (The scale copies once took a barrier
    phase of the wrong stage in this regime: stale scales, then a wait that ran out.) Repeated launches stay
    bit-equal to the first, the two tile widths agree, no wait gives up, and the result is the fp32 product
    of the dequantized operands."""
    from fouroversix_b200 import _native

    m, n, k = 128, 98304, 2880
    g = torch.Generator(device=DEV).manual_seed(2)
    qa = fos.quantize(torch.randn(m, k, generator=g, device=DEV).bfloat16())
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.02).bfloat16()
    qb = fos.quantize(w)
    first = B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, variant=256).clone()
    for _ in range(40):
        assert torch.equal(B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, variant=256), first)
    assert torch.equal(B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, variant=128), first)
    assert _native.wait_failure_site() == 0
    _check(first, _dense_reference(qa, qb), "skinny", mismatch_scale=(k / 1024) ** 0.5)


def test_calls_with_different_options_on_two_streams():
    """Options travel with each call (CTA limit, kernel variant): two GEMMs in flight on two streams
    with different options give the bits each gives alone."""
    g = torch.Generator().manual_seed(11)
    qx = fos.quantize(torch.randn(2048, 1024, generator=g).bfloat16().to(DEV))
    qa = fos.quantize(torch.randn(1536, 1024, generator=g).bfloat16().to(DEV))
    qb = fos.quantize(torch.randn(1024, 1024, generator=g).bfloat16().to(DEV))
    kw_a, kw_b = dict(max_ctas=40), dict(max_ctas=100, variant=128)
    alone_a = B200MatmulBackend.quantized_matmul(qx, qa, out_dtype=fos.DataType.bfloat16, **kw_a).clone()
    alone_b = B200MatmulBackend.quantized_matmul(qx, qb, out_dtype=fos.DataType.bfloat16, **kw_b).clone()
    assert torch.equal(alone_a, B200MatmulBackend.quantized_matmul(qx, qa, out_dtype=fos.DataType.bfloat16))
    cur = torch.cuda.current_stream()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(5):
        s1.wait_stream(cur)
        s2.wait_stream(cur)
        with torch.cuda.stream(s1):
            ya = B200MatmulBackend.quantized_matmul(qx, qa, out_dtype=fos.DataType.bfloat16, **kw_a)
        with torch.cuda.stream(s2):
            yb = B200MatmulBackend.quantized_matmul(qx, qb, out_dtype=fos.DataType.bfloat16, **kw_b)
        cur.wait_stream(s1)
        cur.wait_stream(s2)
        assert torch.equal(ya, alone_a) and torch.equal(yb, alone_b)


@pytest.mark.parametrize("name,m,n,k,rule", [
    ("c2-act-x-weight-static6", 8192, 4096, 4096, "static_6"),
    ("c2-act-x-weight-4over6", 8192, 4096, 4096, "mse"),
    ("c2-square-8192", 8192, 8192, 8192, "mse"),
])
def test_full_size_configs(name, m, n, k, rule):
    g = torch.Generator().manual_seed(1)
    a = torch.randn(m, k, generator=g)
    if "act" in name:
        a[:, torch.randperm(k, generator=g)[: k // 100]] *= 20
        b = torch.randn(n, k, generator=g) * 0.02
    else:
        b = torch.randn(n, k, generator=g)
    cfg = fos.QuantizationConfig(scale_rule=rule)
    qa, qb = fos.quantize(a.bfloat16().to(DEV), cfg), fos.quantize(b.bfloat16().to(DEV), cfg)
    out = B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType.bfloat16, check_status=True)
    _check(out, _dense_reference(qa, qb), name, mismatch_scale=(k / 1024) ** 0.5)
    # linearity in alpha: doubling one operand's amax doubles every output exactly (power of two)
    qa2 = fos.QuantizedTensor(qa.values, qa.scale_factors, qa.amax * 2, qa.dtype, qa.original_shape,
                              qa.scale_rule, qa.round_style, qa.padded_shape)
    out2 = B200MatmulBackend.quantized_matmul(qa2, qb, out_dtype=fos.DataType.bfloat16, check_status=True)
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.parametrize(("name", "m", "n", "k"), [("ragged", 200, 320, 192), ("one-tile", 128, 256, 64),
                                                   ("narrow", 1000, 128, 1024), ("c2-act-x-weight", 8192, 4096, 4096),
                                                   ("c5-qkv", 2048, 10240, 8192)])
@pytest.mark.parametrize("rule", ["static_6", "static_4"])
def test_fused_activation_quantization_equals_the_two_kernels(name, m, n, k, rule):
    """fos_gemm_nvfp4_fused_a quantizes the activation tile by tile inside the GEMM: the output must be
    bit-identical to fos_quantize (same static rule, same amax) followed by fos_gemm_nvfp4 with the same tile
    width, for bf16 and fp16 activations and all three output types."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, k, generator=g)
    x[:, torch.randperm(k, generator=g)[: max(1, k // 100)]] *= 20
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(DEV)
    qw = fos.quantize(w)                                             # 4/6 weights, as in the decoder stack
    cfg = fos.QuantizationConfig(scale_rule=rule)
    for x_dtype, out_dtype in ((torch.bfloat16, "bfloat16"), (torch.float16, "float16"), (torch.bfloat16, "float32")):
        xd = x.to(x_dtype).to(DEV)
        want = B200MatmulBackend.quantized_matmul(fos.quantize(xd, cfg), qw, out_dtype=fos.DataType(out_dtype), check_status=True)
        got = B200MatmulBackend.fused_quantize_matmul(xd, qw, cfg, out_dtype=fos.DataType(out_dtype), check_status=True)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"{name} {rule} {x_dtype} -> {out_dtype}"
        if m > 4096:
            break                                                    # the big shapes once
    # through the front end; a 4/6 activation falls back to the two kernels
    y = fos.quantized_matmul(xd, qw, input_config=cfg, fuse_input_quantization=True, out_dtype=fos.DataType(out_dtype))
    assert torch.equal(y, got)
    y46 = fos.quantized_matmul(xd, qw, fuse_input_quantization=True)
    assert torch.equal(y46, fos.quantized_matmul(xd, qw))
    with pytest.raises(ValueError, match="4/6"):
        B200MatmulBackend.fused_quantize_matmul(xd, qw, fos.QuantizationConfig(), out_dtype=fos.DataType.bfloat16)


# the linear layers of a Llama-3-70B-shaped decoder block (hidden 8192, MLP 28672, grouped-query qkv 10240):
# out features N, in features K; gate_proj and up_proj have the same shape
DECODER_LAYERS = [("qkv_proj", 10240, 8192), ("o_proj", 8192, 8192), ("gate_up_proj", 28672, 8192),
                  ("down_proj", 8192, 28672)]


@pytest.mark.parametrize(("name", "n", "k"), DECODER_LAYERS)
def test_decoder_layer_shapes_against_oracle(oracle, name, n, k):
    """Dynamic 4/6 activation quantization + 4/6 weights + GEMM at the decoder-stack layer shapes, on a
    2048-token slice: packed operands bit for bit against the oracle, the product against the oracle's
    matmul (the reference's 0.1 % bar of tests/test_matmul.py:15, scaled by sqrt(K / 1024) for the longer
    fp32 sums) and within 1e-2 of the fp32 product of the dequantized operands."""
    tokens = 2048
    g = torch.Generator().manual_seed(12 + n + k)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    qx, qw = fos.quantize(x.to(DEV)), fos.quantize(w.to(DEV))
    ox, ow = oracle.quantize(x), oracle.quantize(w)
    for q, o in ((qx, ox), (qw, ow)):
        assert torch.equal(q.values.cpu(), o.values)
        assert torch.equal(q.scale_factors.view(torch.uint8).cpu().flatten(), o.scale_factors)
        assert torch.equal(q.amax.cpu(), o.amax)
    out = B200MatmulBackend.quantized_matmul(qx, qw, out_dtype=fos.DataType.bfloat16, check_status=True)
    _check(out, _dense_reference(qx, qw), name, mismatch_scale=(k / 1024) ** 0.5)
    want = oracle.matmul(ox, ow, torch.bfloat16)
    frac = (out.cpu() != want).float().mean().item()
    assert frac <= MISMATCH_TOLERANCE * (k / 1024) ** 0.5, f"{name} vs oracle matmul: {frac:.3%} differ"


@pytest.mark.parametrize(("m", "n", "k"), [(256, 256, 256), (512, 256, 1024), (100, 72, 80), (384, 640, 448)])
@pytest.mark.parametrize(("dtype_a", "dtype_b"), [("if4", "if4"), ("if4", "nvfp4"), ("nvfp4", "if4")])
def test_if4_matmul_against_oracle(oracle, m, n, k, dtype_a, dtype_b):
    """IF4 operands (and IF4 x NVFP4 mixes) go through the expand-to-fp16 GEMM."""
    g = torch.Generator().manual_seed(17)
    x = torch.randn(m, k, generator=g).bfloat16()
    y = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    ca, cb = fos.QuantizationConfig(dtype=dtype_a), fos.QuantizationConfig(dtype=dtype_b)
    qx, qy = fos.quantize(x.to(DEV), ca), fos.quantize(y.to(DEV), cb)
    out = B200MatmulBackend.quantized_matmul(qx, qy, out_dtype=fos.DataType.bfloat16, check_status=True)
    want = oracle.matmul(oracle.quantize(x, dtype=dtype_a), oracle.quantize(y, dtype=dtype_b), torch.bfloat16)
    torch.cuda.synchronize()
    frac = (out.cpu() != want).float().mean().item()
    assert frac <= MISMATCH_TOLERANCE, f"{frac:.3%} of outputs differ from the oracle"
    _check(out, _dense_reference(qx, qy), f"if4 {m}x{n}x{k} {dtype_a}x{dtype_b}")
    out32 = B200MatmulBackend.quantized_matmul(qx, qy, out_dtype=fos.DataType.float32, check_status=True)
    ref32 = _dense_reference(qx, qy)
    assert ((out32 - ref32).abs().max() / ref32.abs().max()).item() < 1e-5


@pytest.mark.parametrize("name,tokens,k,n", [("c3-up-gate", 4096, 4096, 14336), ("c3-down", 4096, 14336, 4096)])
def test_if4_llama_mlp_shapes(name, tokens, k, n):
    """IF4 quantize + GEMM on Llama-3-8B MLP shapes: Student-t(4)*0.5 activations, N(0, 0.02^2) weights."""
    g = torch.Generator().manual_seed(5)
    z = torch.randn(tokens, k, generator=g)
    chi = (torch.randn(4, tokens, k, generator=g) ** 2).sum(0)
    x = (0.5 * z / (chi / 4).sqrt()).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(DEV)
    cfg = fos.QuantizationConfig(dtype="if4")
    qx, qw = fos.quantize(x, cfg), fos.quantize(w, cfg)
    out = B200MatmulBackend.quantized_matmul(qx, qw, out_dtype=fos.DataType.bfloat16, check_status=True)
    _check(out, _dense_reference(qx, qw), name, mismatch_scale=(k / 1024) ** 0.5)


@pytest.mark.parametrize(("m", "n", "k"), [(256, 256, 256), (512, 1024, 1024), (128, 128, 128), (100, 72, 80),
                                           (130, 300, 384), (384, 640, 448), (1024, 2048, 4096)])
@pytest.mark.parametrize("out_dtype", ["bfloat16", "float32"])
def test_mxfp4_matmul_against_oracle(oracle, m, n, k, out_dtype):
    """MXFP4 x MXFP4 (kind::mxf4, E8M0 scales per 32 values, alpha = 1) against the oracle's matmul of
    the same packed operands and against the fp32 product of the dequantized operands. K values that
    are odd multiples of 128 exercise a last stage with a single scale tile."""
    g = torch.Generator().manual_seed(m + 3 * n + 7 * k)
    a = torch.randn(m, k, generator=g).bfloat16()
    b = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    cfg = fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6")
    qa, qb = fos.quantize(a.to(DEV), cfg), fos.quantize(b.to(DEV), cfg)
    ref32 = _dense_reference(qa, qb)
    for block_n in (128, 256):
        out = B200MatmulBackend.quantized_matmul(qa, qb, out_dtype=fos.DataType(out_dtype), check_status=True, variant=block_n)
        what = f"mxfp4 {m}x{n}x{k} {out_dtype} block_n={block_n}"
        if out_dtype == "float32":
            assert ((out - ref32).abs().max() / ref32.abs().max()).item() < 1e-5, what
        else:
            _check(out, ref32, what, mismatch_scale=max(1.0, (k / 1024) ** 0.5))
    if m * n * k <= 512 * 1024 * 1024 and out_dtype == "bfloat16":
        oa = oracle.quantize(a, dtype="mxfp4", scale_rule="static_6")
        ob = oracle.quantize(b, dtype="mxfp4", scale_rule="static_6")
        want = oracle.matmul(oa, ob, torch.bfloat16)
        assert (out.cpu() != want).float().mean().item() <= MISMATCH_TOLERANCE


def test_mxfp4_golden_matmul_cases():
    import io
    import lzma
    from pathlib import Path

    raw = lzma.decompress((Path(__file__).parent / "golden" / "reference_golden_mxfp4.pt.xz").read_bytes())
    gold = torch.load(io.BytesIO(raw), weights_only=False)
    cfg = fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6")
    for mm in gold["matmuls"]:
        qa, qb = fos.quantize(gold["inputs"][mm["a"]].to(DEV), cfg), fos.quantize(gold["inputs"][mm["b"]].to(DEV), cfg)
        out = fos.quantized_matmul(qa, qb, out_dtype=mm["out_dtype"]).cpu()
        ref = mm["out"]
        rel = ((out.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-30)).item()
        assert rel <= REL_TOLERANCE, (mm["a"], mm["b"], rel)
        if out.dtype == torch.bfloat16:
            assert (out != ref).float().mean().item() <= MISMATCH_TOLERANCE
