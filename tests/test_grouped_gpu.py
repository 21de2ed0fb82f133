"""Grouped quantization and grouped FP4 GEMM (one launch for all experts of a mixture-of-experts layer)
against what they replace: the reference's per-expert loop of quantize + quantized_matmul
(src/fouroversix/model/modules/gpt_oss.py:297-335), run here with the single-problem kernels, which the other
test files pin to the oracle and the golden vectors. Codes, scale bytes, amax and GEMM outputs: bit-exact.
"""

from __future__ import annotations

import pytest
import torch

import fouroversix_b200 as fos
from fouroversix_b200.matmul import GroupLayout, StackedQuantizedTensor, grouped_quantize, grouped_quantized_matmul
from fouroversix_b200.model import FourOverSixExperts
from fouroversix_b200.quantize import to_blocked

pytestmark = pytest.mark.gpu
DEV = "cuda"

COUNTS = {
    "ragged": [5, 0, 300, 128, 1, 0, 77, 257],
    "one-group": [200],
    "empty-ends": [0, 64, 0],
    "many": [((7 * i) % 61) * ((i % 3) != 0) for i in range(48)],
}


def _padded_rows(counts: list[int], k: int, seed: int, dtype=torch.bfloat16):
    """The padded buffer for the given group sizes, every group drawn with a scale of its own (so that the
    groups' amax values differ), and the layout."""
    g = torch.Generator().manual_seed(seed)
    layout = GroupLayout.from_counts(torch.tensor(counts, device=DEV), sum(counts))
    x = torch.zeros(layout.capacity, k, dtype=dtype, device=DEV)
    start = layout.group_start.tolist()
    parts = []
    for i, c in enumerate(counts):
        part = (torch.randn(c, k, generator=g) * (0.25 + i)).to(dtype).to(DEV)
        x[start[i]:start[i] + c] = part
        parts.append(part)
    return x, layout, parts, start


@pytest.mark.parametrize("name", list(COUNTS))
@pytest.mark.parametrize("dtype,rule", [("nvfp4", "mse"), ("nvfp4", "static_6"), ("nvfp4", "mae"), ("if4", "mse")])
def test_grouped_quantize_equals_one_call_per_group(name, dtype, rule):
    counts, k = COUNTS[name], 320
    x, layout, parts, start = _padded_rows(counts, k, seed=len(counts))
    cfg = fos.QuantizationConfig(dtype=dtype, scale_rule=rule)
    gq = grouped_quantize(x, layout, cfg)
    tile_bytes = 128 * k // 16
    for i, c in enumerate(counts):
        if c == 0:
            continue
        want = fos.quantize(parts[i], cfg)
        rows_p = want.padded_shape[0]
        assert torch.equal(gq.amax[i:i + 1], want.amax.reshape(1)), (name, i)
        assert torch.equal(gq.values[start[i]:start[i] + rows_p], want.values), (name, i)
        lo = start[i] // 128 * tile_bytes
        got_sf = gq.scale_factors.view(torch.uint8)[lo:lo + rows_p // 128 * tile_bytes]
        want_sf = want.scale_factors.view(torch.uint8)
        if not want.scale_factors_are_in_blackwell_layout:       # (the single call keeps IF4 scales row-major)
            want_sf = to_blocked(want_sf.reshape(rows_p, k // 16))
        assert torch.equal(got_sf, want_sf.reshape(-1)), (name, i)


def test_grouped_quantize_against_the_oracle():
    from oracle import fos_oracle

    counts, k = [130, 3], 256
    x, layout, parts, start = _padded_rows(counts, k, seed=9, dtype=torch.float16)
    gq = grouped_quantize(x, layout)
    for i, c in enumerate(counts):
        ref = fos_oracle.quantize(parts[i].cpu())
        rows_p = ref.values.shape[0]
        assert torch.equal(gq.amax[i].cpu(), ref.amax.reshape(()))
        assert torch.equal(gq.values[start[i]:start[i] + rows_p].cpu(), ref.values)
        lo = start[i] // 128 * (128 * k // 16)
        assert torch.equal(gq.scale_factors.view(torch.uint8)[lo:lo + ref.scale_factors.numel()].cpu(), ref.scale_factors.reshape(-1))


@pytest.mark.parametrize("name", list(COUNTS))
@pytest.mark.parametrize("n,k,out_dtype,variant", [(384, 320, "bfloat16", 0), (200, 256, "float32", 0),
                                                    (640, 512, "float16", 128), (640, 512, "bfloat16", 256)])
def test_grouped_matmul_equals_one_call_per_group(name, n, k, out_dtype, variant):
    counts = COUNTS[name]
    x, layout, parts, start = _padded_rows(counts, k, seed=3)
    g = torch.Generator().manual_seed(17)
    weights = [(torch.randn(n, k, generator=g) * (0.02 * (1 + i % 5))).bfloat16().to(DEV) for i in range(len(counts))]
    qw = [fos.quantize(w) for w in weights]
    stacked = StackedQuantizedTensor.stack(qw)
    gq = grouped_quantize(x, layout)
    torch_out = getattr(torch, out_dtype)
    canvas = torch.full((layout.capacity, n), 7.0, dtype=torch_out, device=DEV)
    out = grouped_quantized_matmul(gq, stacked, out_dtype=fos.DataType(out_dtype), out=canvas, variant=variant)
    keep = torch.ones(layout.capacity, dtype=torch.bool, device=DEV)
    for i, c in enumerate(counts):
        if c == 0:
            continue
        want = fos.quantized_matmul(fos.quantize(parts[i]), qw[i], out_dtype=fos.DataType(out_dtype))
        assert torch.equal(out[start[i]:start[i] + c], want), (name, i)
        keep[start[i]:start[i] + c] = False
    assert (out[keep] == 7).all(), "rows outside the groups' real rows must not be written"
    from fouroversix_b200 import _native
    assert _native.wait_failure_site() == 0


def test_grouped_matmul_expert_shapes():
    """The shapes of a GPT-OSS expert (hidden 2880, 2 x 2880 gate-up columns), 8 experts, uneven routing."""
    counts, k, n = [700, 0, 33, 1290, 128, 5, 0, 404], 2880, 5760
    x, layout, parts, start = _padded_rows(counts, k, seed=5)
    g = torch.Generator().manual_seed(23)
    qw = [fos.quantize((torch.randn(n, k, generator=g) * 0.02).bfloat16().to(DEV)) for _ in counts]
    out = grouped_quantized_matmul(grouped_quantize(x, layout), StackedQuantizedTensor.stack(qw))
    for i, c in enumerate(counts):
        if c:
            assert torch.equal(out[start[i]:start[i] + c], fos.quantized_matmul(fos.quantize(parts[i]), qw[i])), i


def _reference_style_loop(layer: FourOverSixExperts, hidden, routing_indices, routing_weights):
    """The reference's forward, expert by expert on the host, with the single-problem kernels."""
    down, gate_up = layer.quantized_weights()
    cfg = layer.config.get_activation_config()
    x = hidden.reshape(-1, layer.hidden_size)
    result = torch.zeros_like(x)
    mask = torch.nn.functional.one_hot(routing_indices, num_classes=layer.num_experts).permute(2, 1, 0)
    for e in range(layer.num_experts):
        top_k_pos, token_idx = torch.where(mask[e])
        if token_idx.numel() == 0:
            continue
        gu = fos.quantized_matmul(x[token_idx], gate_up[e], input_config=cfg) + layer.gate_up_proj_bias[e]
        gate, up = gu[..., ::2].clamp(max=layer.limit), gu[..., 1::2].clamp(min=-layer.limit, max=layer.limit)
        gated = (up + 1) * (gate * torch.sigmoid(gate * layer.alpha))
        out = fos.quantized_matmul(gated, down[e], input_config=cfg) + layer.down_proj_bias[e]
        result.index_add_(0, token_idx, (out * routing_weights[token_idx, top_k_pos, None]).to(x.dtype))
    return result.reshape(hidden.shape)


def test_experts_layer_equals_the_per_expert_loop():
    g = torch.Generator().manual_seed(31)
    experts, hidden, inter, tokens, top_k = 8, 256, 192, 300, 2
    layer = FourOverSixExperts(
        (torch.randn(experts, 2 * inter, hidden, generator=g) * 0.05).bfloat16().to(DEV),
        (torch.randn(experts, 2 * inter, generator=g) * 0.1).bfloat16().to(DEV),
        (torch.randn(experts, hidden, inter, generator=g) * 0.05).bfloat16().to(DEV),
        (torch.randn(experts, hidden, generator=g) * 0.1).bfloat16().to(DEV))
    x = torch.randn(2, tokens // 2, hidden, generator=g).bfloat16().to(DEV)
    scores = torch.randn(tokens, experts, generator=g)
    scores[:, 5] = -1e9                                           # an expert nobody is routed to
    weights, indices = torch.topk(torch.softmax(scores, -1), top_k, dim=-1)
    indices, weights = indices.to(DEV), weights.bfloat16().to(DEV)
    got = layer(x, indices, weights)
    want = _reference_style_loop(layer, x, indices, weights)
    # every step is bit-equal group by group, and with two experts per token the two bf16 additions into a
    # token's row commute: the whole layer is bit-equal
    assert (got.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
    assert torch.equal(got, want)
