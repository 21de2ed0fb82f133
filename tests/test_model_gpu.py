"""`FourOverSixLinear` and `quantize_model` on the GPU: forward, backward, packed buffers.

The layer only orchestrates `quantize` and `quantized_matmul` (both checked against the
oracle elsewhere), so these tests check the orchestration: which operand is quantized how,
which transposes are taken, that the packed state dict round-trips, and that the result is
what the reference's formulas give when evaluated with dequantized operands.
"""

from __future__ import annotations

import pytest
import torch
import torch.nn as nn

import fouroversix_b200 as fos

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _fp32_matmul(a, b):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return a.float() @ b.float()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def _close(out, ref32, tol=1e-2):
    rel = ((out.float() - ref32).abs().max() / ref32.abs().max().clamp_min(1e-30)).item()
    assert rel <= tol, rel


def test_ptq_linear_forward_matches_dequantized_matmul():
    torch.manual_seed(0)
    lin = nn.Linear(512, 384, bias=True, device=DEV, dtype=torch.bfloat16)
    w, b = lin.weight.data.clone(), lin.bias.data.clone()
    q = fos.FourOverSixLinear(lin, fos.ModuleQuantizationConfig()).quantize_weight_()
    assert q.weight is None and int(q.quantized_weight_metadata[0]) == 384
    x = torch.randn(3, 40, 512, device=DEV, dtype=torch.bfloat16)
    y = q(x)
    assert y.shape == (3, 40, 384) and y.dtype == torch.bfloat16
    xq = fos.dequantize(fos.quantize(x.reshape(-1, 512)), torch.float32)
    wq = fos.dequantize(fos.quantize(w), torch.float32)
    ref = (_fp32_matmul(xq, wq.T) + b.float()).reshape(3, 40, 384)
    _close(y, ref)
    assert torch.equal(q.dequantized_weight(torch.float32), wq)


@pytest.mark.parametrize("shape,k,n,rule,out", [((16,), 8192, 8192, "mse", "bfloat16"), ((3, 41), 520, 392, "static_6", "float16"),
                                                ((300,), 1024, 2880, "mae", "float32")])
def test_one_call_forward_equals_the_call_by_call_forward(shape, k, n, rule, out):
    """Inference on a packed weight takes `fos_linear_forward` (one host call); the autograd function quantizes and
    multiplies call by call. Same kernels, same bits - ragged rows, a width that is not a multiple of 64, a bias."""
    from fouroversix_b200.model.linear import FourOverSixLinearFunction

    torch.manual_seed(1)
    lin = nn.Linear(k, n, bias=True, device=DEV, dtype=torch.bfloat16)
    cfg = fos.ModuleQuantizationConfig(scale_rule=rule, output_dtype=out)
    q = fos.FourOverSixLinear(lin, cfg).quantize_weight_()
    x = torch.randn(*shape, k, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        assert q._one_call_forward_applies(x)
        got = q(x)
        want = FourOverSixLinearFunction.apply(cfg, x, q.quantized_weight(), q.bias)
    assert got.shape == (*shape, n) and got.dtype == want.dtype
    assert torch.equal(got, want)
    # an input that needs a gradient goes through the autograd function
    assert not q._one_call_forward_applies(x.clone().requires_grad_())


def test_packed_state_dict_round_trips_between_modules():
    torch.manual_seed(1)
    src = fos.FourOverSixLinear(nn.Linear(256, 128, bias=False, device=DEV, dtype=torch.bfloat16),
                                fos.ModuleQuantizationConfig(scale_rule="static_6")).quantize_weight_()
    sd = {k: v for k, v in src.state_dict().items() if k.startswith("quantized_")}
    assert set(sd) == {"quantized_weight_values", "quantized_weight_scale_factors", "quantized_weight_amax",
                       "quantized_weight_metadata"}
    dst = fos.FourOverSixLinear(nn.Linear(256, 128, bias=False, device=DEV, dtype=torch.bfloat16),
                                fos.ModuleQuantizationConfig(scale_rule="static_6"))
    dst.weight = None
    dst.load_state_dict(sd, strict=False)
    x = torch.randn(64, 256, device=DEV, dtype=torch.bfloat16)
    assert torch.equal(src(x), dst(x))


def test_quantize_model_on_a_small_mlp_stack():
    torch.manual_seed(2)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.up, self.gate, self.down = nn.Linear(256, 512, bias=False), nn.Linear(256, 512, bias=False), \
                nn.Linear(512, 256, bias=False)

        def forward(self, x):
            return self.down(torch.nn.functional.silu(self.gate(x)) * self.up(x))

    model = nn.Sequential(Block(), Block()).to(DEV, torch.bfloat16)
    model.add_module("lm_head", nn.Linear(256, 100, bias=False, device=DEV, dtype=torch.bfloat16))
    x = torch.randn(2, 128, 256, device=DEV, dtype=torch.bfloat16)
    want = model(x)
    fos.quantize_model(model, fos.ModelQuantizationConfig(keep_master_weights=True))
    assert all(isinstance(m, fos.FourOverSixLinear) for m in (model[0].up, model[0].gate, model[0].down, model[1].down))
    assert not isinstance(model.lm_head, fos.FourOverSixLinear)
    got = model(x)
    # FP4 on both operands of six GEMMs and two gated non-linearities: the output keeps its direction
    # (cosine similarity) but carries tens of percent of quantization noise
    cos = torch.nn.functional.cosine_similarity(got.float().flatten(), want.float().flatten(), dim=0).item()
    assert cos > 0.85, cos
    assert torch.isfinite(got.float()).all()


@pytest.mark.parametrize("tokens,k,n", [(256, 256, 384), (4096, 4096, 4096)])
def test_training_forward_dgrad_wgrad(tokens, k, n):
    """keep_master_weights + 2-D weight blocks + nearest gradient rounding: the three FP4 GEMMs of a
    step equal the formulas evaluated on dequantized operands (the transposed quantizations included)."""
    g = torch.Generator().manual_seed(9)
    x = torch.randn(1, tokens, k, generator=g).bfloat16().to(DEV).requires_grad_(True)
    lin = nn.Linear(k, n, bias=False, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        lin.weight.copy_((torch.randn(n, k, generator=g) * 0.02).bfloat16())
    dy = (torch.randn(1, tokens, n, generator=g) * 1e-3).bfloat16().to(DEV)
    cfg = fos.ModuleQuantizationConfig(keep_master_weights=True, weight_scale_2d=True, gradient_round_style="nearest")
    layer = fos.FourOverSixLinear(lin, cfg)
    y = layer(x)
    y.backward(dy)

    x2, dy2, w = x.detach().reshape(tokens, k), dy.reshape(tokens, n), lin.weight.data
    deq = lambda t, **c: fos.dequantize(fos.quantize(t, fos.QuantizationConfig(**c)), torch.float32)  # noqa: E731
    w_q = deq(w, block_scale_2d=True)
    _close(y.reshape(tokens, n), _fp32_matmul(deq(x2), w_q.T))
    # dgrad: q(dy) @ q(W^T)^T ; with 16x16 blocks q(W^T) == q(W)^T
    wt_q = deq(w, block_scale_2d=True, transpose=True)
    assert torch.equal(wt_q, w_q.T)
    _close(x.grad.reshape(tokens, k), _fp32_matmul(deq(dy2), wt_q.T))
    # wgrad: q(rot(dy^T)) @ q(rot(x^T))^T: both operands rotated along the token axis by the same
    # orthogonal transform, as in the reference
    _close(lin.weight.grad, _fp32_matmul(deq(dy2, transpose=True, rht=True), deq(x2, transpose=True, rht=True).T))
    # and the rotation leaves the product itself alone: the result is the true gradient up to FP4 noise
    true = _fp32_matmul(dy2.T, x2)
    cos = torch.nn.functional.cosine_similarity(lin.weight.grad.float().flatten(), true.flatten(), dim=0).item()
    assert cos > 0.97, cos


def test_default_backward_uses_stochastic_gradient_rounding():
    """The reference's defaults: gradients rounded stochastically (seeded from torch's CPU generator),
    wgrad operands rotated. Repeatable under torch.manual_seed, different across seeds, unbiased enough
    that the gradients keep the direction of the exact ones."""
    g = torch.Generator().manual_seed(3)
    lin = nn.Linear(512, 256, bias=False, device=DEV, dtype=torch.bfloat16)
    layer = fos.FourOverSixLinear(lin, fos.ModuleQuantizationConfig(keep_master_weights=True))
    x0 = torch.randn(1, 1024, 512, generator=g).bfloat16().to(DEV)
    dy = (torch.randn(1, 1024, 256, generator=g) * 1e-3).bfloat16().to(DEV)

    def grads(seed):
        torch.manual_seed(seed)
        x = x0.clone().requires_grad_(True)
        lin.weight.grad = None
        layer(x).backward(dy)
        return x.grad.clone(), lin.weight.grad.clone()

    dx_a, dw_a = grads(1)
    dx_b, dw_b = grads(1)
    dx_c, dw_c = grads(2)
    assert torch.equal(dx_a, dx_b) and torch.equal(dw_a, dw_b)
    assert not torch.equal(dx_a, dx_c) and not torch.equal(dw_a, dw_c)
    true_dx = _fp32_matmul(dy.reshape(-1, 256), lin.weight.data).reshape(1, 1024, 512)
    true_dw = _fp32_matmul(dy.reshape(-1, 256).T, x0.reshape(-1, 512))
    for got, true in ((dx_a, true_dx), (dw_a, true_dw)):
        cos = torch.nn.functional.cosine_similarity(got.float().flatten(), true.flatten(), dim=0).item()
        assert cos > 0.95, cos


def test_unbiased_stochastic_rounding_backward():
    """gradient_round_style="stochastic_unbiased": the gradients' scale factors are computed against
    16/17 of the format's range and the factor is undone in the GEMM's alpha, so the backward GEMMs
    still estimate the true products (reference: quantize/reference.py:331-343, 430-440)."""
    g = torch.Generator().manual_seed(4)
    lin = nn.Linear(512, 256, bias=False, device=DEV, dtype=torch.bfloat16)
    layer = fos.FourOverSixLinear(
        lin, fos.ModuleQuantizationConfig(keep_master_weights=True, gradient_round_style="stochastic_unbiased"))
    x0 = torch.randn(1, 1024, 512, generator=g).bfloat16().to(DEV)
    dy = (torch.randn(1, 1024, 256, generator=g) * 1e-3).bfloat16().to(DEV)
    torch.manual_seed(1)
    x = x0.clone().requires_grad_(True)
    layer(x).backward(dy)
    true_dx = _fp32_matmul(dy.reshape(-1, 256), lin.weight.data).reshape(1, 1024, 512)
    true_dw = _fp32_matmul(dy.reshape(-1, 256).T, x0.reshape(-1, 512))
    for got, true in ((x.grad, true_dx), (lin.weight.grad, true_dw)):
        cos = torch.nn.functional.cosine_similarity(got.float().flatten(), true.flatten(), dim=0).item()
        ratio = (got.float().norm() / true.norm()).item()
        assert cos > 0.95, cos
        assert 0.9 < ratio < 1.1, ratio


def test_mxfp4_linear_forward():
    """The same layer with the reference's second format: dtype="mxfp4", static_6 (the only kind of
    rule the format defines). Forward = q(x) @ q(W)^T with alpha = 1."""
    g = torch.Generator().manual_seed(5)
    lin = nn.Linear(512, 384, bias=True, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(2, 100, 512, generator=g).bfloat16().to(DEV)
    cfg = fos.ModuleQuantizationConfig(dtype="mxfp4", scale_rule="static_6")
    w = lin.weight.data.clone()
    layer = fos.FourOverSixLinear(lin, cfg).quantize_weight_()
    assert layer.quantized_weight_scale_factors.dtype == torch.float8_e8m0fnu
    assert layer.quantized_weight_scale_factors.numel() == 384 * 512 // 32
    out = layer(x)
    qc = fos.QuantizationConfig(dtype="mxfp4", scale_rule="static_6")
    xq = fos.dequantize(fos.quantize(x.reshape(-1, 512), qc), torch.float32)
    wq = fos.dequantize(fos.quantize(w, qc), torch.float32)
    want = (_fp32_matmul(xq, wq.T) + layer.bias.float()).reshape(2, 100, 384)
    _close(out, want)
