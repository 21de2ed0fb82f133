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
        od = layer.config.output_dtype
        gu = fos.quantized_matmul(x[token_idx], gate_up[e], input_config=cfg, out_dtype=od) + layer.gate_up_proj_bias[e]
        gate, up = gu[..., ::2].clamp(max=layer.limit), gu[..., 1::2].clamp(min=-layer.limit, max=layer.limit)
        gated = (up + 1) * (gate * torch.sigmoid(gate * layer.alpha))
        out = fos.quantized_matmul(gated, down[e], input_config=cfg, out_dtype=od) + layer.down_proj_bias[e]
        result.index_add_(0, token_idx, (out * routing_weights[token_idx, top_k_pos, None]).to(x.dtype))
    return result.reshape(hidden.shape)


def _experts_case(seed, experts, hidden, inter, tokens, top_k, dtype=torch.bfloat16, **kwargs):
    from fouroversix_b200.model.config import ModuleQuantizationConfig
    from fouroversix_b200.utils import DataType

    g = torch.Generator().manual_seed(seed)
    cfg = ModuleQuantizationConfig(output_dtype=DataType.bfloat16 if dtype == torch.bfloat16 else DataType.float16)
    layer = FourOverSixExperts(
        (torch.randn(experts, 2 * inter, hidden, generator=g) * 0.05).to(dtype).to(DEV),
        (torch.randn(experts, 2 * inter, generator=g) * 0.1).to(dtype).to(DEV),
        (torch.randn(experts, hidden, inter, generator=g) * 0.05).to(dtype).to(DEV),
        (torch.randn(experts, hidden, generator=g) * 0.1).to(dtype).to(DEV), cfg, **kwargs)
    x = torch.randn(2, tokens // 2, hidden, generator=g).to(dtype).to(DEV)
    scores = torch.randn(tokens, experts, generator=g)
    scores[:, min(5, experts - 1)] = -1e9                         # an expert nobody is routed to
    weights, indices = torch.topk(torch.softmax(scores, -1), top_k, dim=-1)
    return layer, x, indices.to(DEV), weights.to(dtype).to(DEV)


@pytest.mark.parametrize("how", [dict(), dict(single_call=False), dict(native_elementwise=False)],
                         ids=["one-call", "kernels", "tensor-ops"])
def test_experts_layer_equals_the_per_expert_loop(how):
    """fos_experts_forward; the same kernels called one by one; the element-wise steps as tensor operations."""
    layer, x, indices, weights = _experts_case(31, 8, 256, 192, 300, 2, **how)
    got = layer(x, indices, weights)
    want = _reference_style_loop(layer, x, indices, weights)
    # every step is bit-equal group by group, and with two experts per token the two 16-bit additions into a
    # token's row commute: the whole layer is bit-equal in either form
    assert (got.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_experts_layer_four_experts_per_token(dtype):
    """With more than two experts per token the order of the additions into a token's row matters: the combine
    kernel adds in ascending order of the expert, as the host loop does (whose index_add_ calls are one per
    expert), so the layer stays bit-equal. GPT-OSS widths (2880: a multiple of 8, not of 128)."""
    layer, x, indices, weights = _experts_case(37, 12, 2880, 2880, 96, 4, dtype)
    got = layer(x, indices, weights)
    want = _reference_style_loop(layer, x, indices, weights)
    assert torch.equal(got, want)


def _op_chain_glu(gu, bias, alpha, limit):
    gu = gu + bias
    gate, up = gu[..., ::2].clamp(min=None, max=limit), gu[..., 1::2].clamp(min=-limit, max=limit)
    return (up + 1) * (gate * torch.sigmoid(gate * alpha))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_glu_kernel_keeps_every_rounding_of_the_operation_chain(dtype):
    """fos_experts_glu against the chain of tensor operations it replaces, on every 16-bit gate value there is
    (so every rounding of the sigmoid is seen), and on limits and factors that are not 16-bit numbers."""
    from fouroversix_b200 import _native

    bits = torch.arange(-32768, 32768, dtype=torch.int32).to(torch.int16).to(DEV)
    gates = bits.view(dtype)                                      # all 65536 patterns: NaNs, infinities, subnormals
    g = torch.Generator().manual_seed(3)
    ups = (torch.randn(65536, generator=g) * 4).to(dtype).to(DEV)
    rows, inter = 128, 512
    gu = torch.stack([gates, ups], dim=1).reshape(rows, 2 * inter).contiguous()
    bias = (torch.randn(3, 2 * inter, generator=g) * 0.5).to(dtype).to(DEV)
    bias[0] = 0
    row_expert = (torch.arange(rows, device=DEV) % 4 - 1).to(torch.int32)          # -1: a padding row
    # alpha = 1 with no bias and no effective limit feeds every 16-bit pattern to the sigmoid itself (expert 0)
    for alpha, limit in ((1.702, 7.0), (0.3333, 2.7182818), (1.0, 3.0e38)):
        if alpha == 1.0:
            bias.zero_()
        out = torch.full((rows, inter), 9, dtype=dtype, device=DEV)
        amax = torch.zeros(3, dtype=torch.float32, device=DEV)
        _native.check(_native.lib().fos_experts_glu(gu.data_ptr(), _native.elem_code(dtype), gu.stride(0), bias.data_ptr(),
                                                    row_expert.data_ptr(), out.data_ptr(), out.stride(0), rows, inter,
                                                    alpha, limit, amax.data_ptr(), _native.stream_ptr(gu.device)), "fos_experts_glu")
        real = row_expert >= 0
        want = _op_chain_glu(gu[real], bias[row_expert[real].long()], alpha, limit)
        assert (out[~real] == 0).all()
        got = out[real]
        same = (got == want) | (got.isnan() & want.isnan())
        assert same.all(), (alpha, limit, int((~same).sum()))
        for e in range(3):                                        # the per-expert maxima, NaNs skipped
            mine = out[row_expert == e].float().abs()
            assert amax[e].item() == mine[~mine.isnan()].max().item()


def test_gather_and_combine_kernels():
    """fos_experts_gather_rows and fos_experts_combine against index operations, slots listed in any order."""
    from fouroversix_b200 import _native

    g = torch.Generator().manual_seed(9)
    tokens, top_k, hidden, experts, cap = 50, 3, 136, 6, 512
    lib, code = _native.lib(), _native.FOS_BF16
    x = torch.randn(tokens, hidden, generator=g).bfloat16().to(DEV)
    row_token = torch.full((cap,), -1, dtype=torch.int32)
    rows = torch.randperm(cap, generator=g)[:tokens * top_k]
    row_token[rows] = (torch.arange(tokens * top_k) // top_k).to(torch.int32)
    row_token = row_token.to(DEV)
    out = torch.full((cap, hidden), 5, dtype=torch.bfloat16, device=DEV)
    row_expert = torch.where(row_token >= 0, row_token % experts, row_token)
    amax = torch.zeros(experts, dtype=torch.float32, device=DEV)
    _native.check(lib.fos_experts_gather_rows(x.data_ptr(), code, x.stride(0), row_token.data_ptr(), out.data_ptr(),
                                              out.stride(0), cap, hidden, row_expert.data_ptr(), amax.data_ptr(),
                                              _native.stream_ptr(x.device)), "gather")
    want = torch.where(row_token[:, None] >= 0, x[row_token.clamp(min=0).long()], torch.zeros_like(out))
    assert torch.equal(out, want)
    for e in range(experts):
        assert amax[e].item() == want[row_expert == e].float().abs().max().item()
    out2 = torch.empty_like(out)
    _native.check(lib.fos_experts_gather_rows(x.data_ptr(), code, x.stride(0), row_token.data_ptr(), out2.data_ptr(),
                                              out2.stride(0), cap, hidden, 0, 0, _native.stream_ptr(x.device)), "gather")
    assert torch.equal(out2, want)

    y = torch.randn(cap, hidden, generator=g).bfloat16().to(DEV)
    bias = torch.randn(experts, hidden, generator=g).bfloat16().to(DEV)
    pair_expert = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).to(torch.int32).to(DEV)
    pair_row = rows.to(torch.int32).to(DEV)
    weight = torch.rand(tokens * top_k, generator=g).bfloat16().to(DEV)
    got = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=DEV)
    _native.check(lib.fos_experts_combine(y.data_ptr(), code, y.stride(0), bias.data_ptr(), pair_row.data_ptr(),
                                          pair_expert.data_ptr(), weight.data_ptr(), top_k, got.data_ptr(), got.stride(0),
                                          tokens, hidden, _native.stream_ptr(x.device)), "combine")
    want = torch.zeros(tokens, hidden, dtype=torch.bfloat16, device=DEV)
    flat_e, token = pair_expert.reshape(-1).long(), torch.arange(tokens * top_k, device=DEV) // top_k
    for e in range(experts):                                      # ascending experts, one 16-bit addition each
        sel = (flat_e == e).nonzero().reshape(-1)
        want.index_add_(0, token[sel], (y[pair_row[sel].long()] + bias[e]) * weight[sel, None])
    assert torch.equal(got, want)


@pytest.mark.parametrize("index_dtype", [torch.int64, torch.int32], ids=["int64", "int32"])
@pytest.mark.parametrize("tokens,top_k,experts", [(300, 2, 8), (8192, 4, 32), (5, 1, 256), (1500, 8, 13)])
def test_route_kernel_tables(tokens, top_k, experts, index_dtype):
    """fos_experts_route against counts, a padded running sum and the definition of its tables."""
    g = torch.Generator().manual_seed(tokens + experts)
    scores = torch.rand(tokens, experts, generator=g)
    if experts > 2:
        scores[:, 1] = -1                                         # an expert nobody is routed to
    indices = torch.topk(scores, top_k, dim=-1).indices.to(index_dtype).to(DEV)
    layer = FourOverSixExperts.__new__(FourOverSixExperts)
    torch.nn.Module.__init__(layer)
    layer.num_experts = experts
    layout, row_token, row_expert, pair_row, pair_expert = layer.route_native(indices)
    flat = indices.reshape(-1).long()
    counts = torch.bincount(flat, minlength=experts)
    assert torch.equal(layout.group_rows.long(), counts)
    padded = (counts + 127) // 128 * 128
    assert torch.equal(layout.group_start.long(), torch.cat([torch.zeros(1, dtype=torch.int64, device=DEV), padded.cumsum(0)]))
    assert layout.capacity % 128 == 0 and layout.capacity >= int(padded.sum())
    assert torch.equal(pair_expert.long(), flat)
    rows = pair_row.long()
    start = layout.group_start.long()[flat]
    assert ((rows >= start) & (rows < start + counts[flat])).all()
    assert rows.unique().numel() == rows.numel()
    assert torch.equal(row_expert[rows].long(), flat)
    assert torch.equal(row_token[rows].long(), torch.arange(flat.numel(), device=DEV) // top_k)
    other = torch.ones(layout.capacity, dtype=torch.bool, device=DEV)
    other[rows] = False
    assert (row_token[other] == -1).all() and (row_expert[other] == -1).all()
    for e in range(experts):                                      # stable: ascending pairs get ascending rows
        mine = rows[flat == e]
        assert (mine[1:] > mine[:-1]).all()
