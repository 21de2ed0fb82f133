"""FP4 experts of a mixture-of-experts layer on the grouped kernels.

The arithmetic of the reference's GPT-OSS experts module (src/fouroversix/model/modules/gpt_oss.py:270-335):
per expert, quantize the routed tokens as one tensor, `quantized_matmul` with the expert's gate-up weight, bias,
clamped SwiGLU, quantize again, `quantized_matmul` with the down weight, bias, weight by the routing score and
add into the token's output row. The reference walks the experts in a host loop and reads the routed indices
back from the device for each; here the routed rows are sorted by expert on the device, laid out in one padded
buffer, and each of the two projections is one grouped quantize launch and one grouped GEMM launch for all
experts. Nothing is read back, so the layer can be captured in a CUDA graph.

Buffers carry the reference's names (`quantized_{gate_up,down}_proj_{values,scale_factors,amax,metadata}`,
src/fouroversix/model/modules/gpt_oss.py:108-196) so that a packed checkpoint loads into either.
"""

from __future__ import annotations

import torch
from torch import nn

from fouroversix_b200 import _native
from fouroversix_b200.matmul.grouped import (_OUT, GroupLayout, StackedQuantizedTensor, grouped_quantize,
                                             grouped_quantized_matmul)
from fouroversix_b200.quantize import quantize
from fouroversix_b200.utils import DataType, RoundStyle, ScaleRule

from .config import ModuleQuantizationConfig


class FourOverSixExperts(nn.Module):
    """`gate_up_proj` [experts, 2 * intermediate, hidden] and `down_proj` [experts, hidden, intermediate] in the
    (out_features, in_features) orientation the reference stores them in after quantization; biases
    [experts, 2 * intermediate] and [experts, hidden]. Gate and up columns are interleaved (even / odd), as in
    the reference."""

    def __init__(self, gate_up_proj: torch.Tensor, gate_up_proj_bias: torch.Tensor, down_proj: torch.Tensor,
                 down_proj_bias: torch.Tensor, config: ModuleQuantizationConfig | None = None, *,
                 alpha: float = 1.702, limit: float = 7.0, native_elementwise: bool = True, single_call: bool = True) -> None:
        super().__init__()
        self.native_elementwise = native_elementwise
        self.single_call = single_call            # fos_experts_forward where the shapes allow; else one call per kernel
        self.config = config or ModuleQuantizationConfig()
        if DataType(self.config.dtype) != DataType.nvfp4:
            raise NotImplementedError("the grouped kernels take nvfp4 operands")
        self.num_experts, two_i, self.hidden_size = gate_up_proj.shape
        self.intermediate_size = two_i // 2
        if down_proj.shape != (self.num_experts, self.hidden_size, self.intermediate_size):
            raise ValueError("down_proj must be [experts, hidden, intermediate]")
        self.alpha, self.limit = alpha, limit
        self.gate_up_proj_bias = nn.Parameter(gate_up_proj_bias.detach().clone(), requires_grad=False)
        self.down_proj_bias = nn.Parameter(down_proj_bias.detach().clone(), requires_grad=False)
        weight_config = self.config.get_weight_config()
        for prefix, weight in (("gate_up", gate_up_proj), ("down", down_proj)):
            tensors = [quantize(weight[e].contiguous(), weight_config) for e in range(self.num_experts)]
            stacked = StackedQuantizedTensor.stack(tensors)
            self.register_buffer(f"quantized_{prefix}_proj_values", stacked.values)
            self.register_buffer(f"quantized_{prefix}_proj_scale_factors", stacked.scale_factors)
            self.register_buffer(f"quantized_{prefix}_proj_amax", stacked.amax.reshape(-1, 1))
            meta = torch.tensor([[*stacked.original_shape, *stacked.padded_shape, 1, 1]] * self.num_experts, dtype=torch.int32)
            self.register_buffer(f"quantized_{prefix}_proj_metadata", meta.to(weight.device))

    def quantized_weights(self) -> tuple[StackedQuantizedTensor, StackedQuantizedTensor]:
        """(down, gate_up), the order of the reference's method of the same name."""
        rule = self.config.get_weight_config().scale_rule
        out = []
        for prefix in ("down", "gate_up"):
            shape = (self.hidden_size, self.intermediate_size) if prefix == "down" else (2 * self.intermediate_size, self.hidden_size)
            values = getattr(self, f"quantized_{prefix}_proj_values")
            padded = (values.shape[1], values.shape[2] * 2)
            out.append(StackedQuantizedTensor(values, getattr(self, f"quantized_{prefix}_proj_scale_factors"),
                                              getattr(self, f"quantized_{prefix}_proj_amax").reshape(-1),
                                              DataType.nvfp4, rule, shape, padded))
        return out[0], out[1]

    def route(self, routing_indices: torch.Tensor) -> tuple[GroupLayout, torch.Tensor, torch.Tensor, torch.Tensor]:
        """Sorts the (token, slot) pairs by expert on the device. Returns the row layout, for every sorted pair
        its row in the padded buffer, its token and its position in the flattened routing tensors."""
        tokens, top_k = routing_indices.shape
        flat = routing_indices.reshape(-1)
        pairs = flat.numel()
        counts = torch.zeros(self.num_experts, dtype=torch.int64, device=flat.device)
        counts.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.int64))
        layout = GroupLayout.from_counts(counts, pairs)
        # the radix sort makes one pass per byte of the key: sort the narrowest type that holds an expert's index
        key = torch.uint8 if self.num_experts <= 256 else torch.int16 if self.num_experts <= 32768 else torch.int32
        order = torch.argsort(flat.to(key), stable=True)
        expert = flat[order]
        first = torch.cumsum(counts, 0) - counts                          # first sorted position of each expert
        rows = layout.group_start.to(torch.int64)[expert] + (torch.arange(pairs, device=flat.device) - first[expert])
        return layout, rows, order // top_k, order

    def forward(self, hidden_states: torch.Tensor, routing_indices: torch.Tensor, routing_weights: torch.Tensor) -> torch.Tensor:
        """hidden_states [batch, seq, hidden] (or [tokens, hidden]); routing_indices / routing_weights
        [tokens, top_k]: the experts each token goes to and the weight of each."""
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_size)
        down, gate_up = self.quantized_weights()
        act_config = self.config.get_activation_config()
        out_dtype = self.config.output_dtype
        if self._native_elementwise(x, routing_weights, out_dtype):
            return self._forward_native(x, routing_indices, routing_weights).reshape(shape)

        layout, rows, token, order = self.route(routing_indices)
        expert = routing_indices.reshape(-1)[order]
        padded = torch.zeros(layout.capacity, self.hidden_size, dtype=x.dtype, device=x.device)
        padded[rows] = x[token]
        gu = grouped_quantized_matmul(grouped_quantize(padded, layout, act_config), gate_up, out_dtype=out_dtype)
        gu = gu[rows] + self.gate_up_proj_bias[expert]
        gate, up = gu[..., ::2], gu[..., 1::2]
        gate = gate.clamp(min=None, max=self.limit)
        up = up.clamp(min=-self.limit, max=self.limit)
        gated = (up + 1) * (gate * torch.sigmoid(gate * self.alpha))

        padded2 = torch.zeros(layout.capacity, self.intermediate_size, dtype=x.dtype, device=x.device)
        padded2[rows] = gated.to(x.dtype)
        y = grouped_quantized_matmul(grouped_quantize(padded2, layout, act_config), down, out_dtype=out_dtype)
        y = (y[rows] + self.down_proj_bias[expert]) * routing_weights.reshape(-1)[order, None]
        result = torch.zeros_like(x)
        result.index_add_(0, token, y.to(x.dtype))
        return result.reshape(shape)

    def _native_elementwise(self, x: torch.Tensor, routing_weights: torch.Tensor, out_dtype: DataType) -> bool:
        """The three element-wise kernels take 16-bit tensors of one type, widths that are multiples of 8 and at
        most 8 experts per token; anything else runs the same arithmetic as tensor operations."""
        if not self.native_elementwise:
            return False
        same = x.dtype == _OUT[DataType(out_dtype)] == routing_weights.dtype == self.gate_up_proj_bias.dtype == self.down_proj_bias.dtype
        return (same and x.dtype in (torch.bfloat16, torch.float16) and self.hidden_size % 8 == 0
                and self.intermediate_size % 8 == 0 and routing_weights.shape[-1] <= 8)

    def route_native(self, routing_indices: torch.Tensor) -> tuple[GroupLayout, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """`fos_experts_route`: the row layout and the tables of the element-wise kernels (row -> token, row ->
        expert, pair -> row, pair -> expert) in two launches."""
        tokens, top_k = routing_indices.shape
        dev = routing_indices.device
        if routing_indices.dtype not in (torch.int32, torch.int64):
            routing_indices = routing_indices.to(torch.int64)
        routing_indices = routing_indices.contiguous()
        capacity = (tokens * top_k + 127 * self.num_experts + 127) // 128 * 128
        work = _native.EXPERTS_ROUTE_WORKSPACE_INTS * self.num_experts
        tables = torch.empty(2 * self.num_experts + 1 + 2 * capacity + 2 * tokens * top_k + work, dtype=torch.int32, device=dev)
        group_start, group_rows, row_token, row_expert, pair_row, pair_expert, workspace = torch.split(
            tables, [self.num_experts + 1, self.num_experts, capacity, capacity, tokens * top_k, tokens * top_k, work])
        _native.check(_native.lib().fos_experts_route(
            routing_indices.data_ptr(), routing_indices.element_size(), tokens, top_k, self.num_experts, capacity,
            group_start.data_ptr(), group_rows.data_ptr(), row_token.data_ptr(), row_expert.data_ptr(),
            pair_row.data_ptr(), pair_expert.data_ptr(), workspace.data_ptr(), _native.stream_ptr(dev)), "fos_experts_route")
        return GroupLayout(group_start, group_rows, capacity, self.num_experts), row_token, row_expert, pair_row, pair_expert

    def _forward_native(self, x: torch.Tensor, routing_indices: torch.Tensor, routing_weights: torch.Tensor) -> torch.Tensor:
        """The same layer on `fos_experts_route`, `fos_experts_gather_rows`, `fos_experts_glu` and
        `fos_experts_combine` around the grouped launches (eleven kernels in all): bit-equal to the
        tensor-operation form when a token has at most two experts, and to the reference's host loop (which adds
        a token's experts in ascending order) for any number."""
        down, gate_up = self.quantized_weights()
        act_config = self.config.get_activation_config()
        out_dtype = self.config.output_dtype
        dev, dtype, code = x.device, x.dtype, _native.elem_code(x.dtype)
        tokens, top_k = routing_indices.shape
        x = x if x.stride(-1) == 1 else x.contiguous()
        with torch.cuda.device(dev):
            return self._run_native(x, routing_indices, routing_weights, down, gate_up, act_config, out_dtype, dev, dtype,
                                    code, tokens, top_k)

    def _run_native(self, x, routing_indices, routing_weights, down, gate_up, act_config, out_dtype, dev, dtype, code,
                    tokens, top_k) -> torch.Tensor:
        lib, stream = _native.lib(), _native.stream_ptr(dev)
        if (self.single_call and self.hidden_size % 64 == 0 and self.intermediate_size % 64 == 0
                and DataType(act_config.dtype) == DataType.nvfp4 and not act_config.block_scale_2d and not act_config.rht
                and RoundStyle(act_config.round_style) == RoundStyle.nearest):
            # one host call for the eleven launches (fos_experts_forward); the workspace is the call's only scratch
            if routing_indices.dtype not in (torch.int32, torch.int64):
                routing_indices = routing_indices.to(torch.int64)
            routing_indices = routing_indices.contiguous()
            weights = routing_weights.reshape(-1).contiguous()
            gate_up_bias, down_bias = self.gate_up_proj_bias.contiguous(), self.down_proj_bias.contiguous()
            need = lib.fos_experts_workspace_bytes(tokens, top_k, self.num_experts, self.hidden_size, self.intermediate_size)
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
            result = torch.empty(tokens, self.hidden_size, dtype=dtype, device=dev)
            _native.check(lib.fos_experts_forward(
                x.data_ptr(), code, tokens, self.hidden_size, x.stride(0), routing_indices.data_ptr(),
                routing_indices.element_size(), weights.data_ptr(), top_k, self.num_experts,
                gate_up.values.data_ptr(), gate_up.scale_factors.data_ptr(), gate_up.amax.data_ptr(), gate_up_bias.data_ptr(),
                down.values.data_ptr(), down.scale_factors.data_ptr(), down.amax.data_ptr(), down_bias.data_ptr(),
                self.intermediate_size, gate_up.scale_rule.cuda_id, ScaleRule(act_config.scale_rule).cuda_id,
                float(self.alpha), float(self.limit), result.data_ptr(), result.stride(0), workspace.data_ptr(), need, 0,
                stream), "fos_experts_forward")
            return result
        layout, row_token, row_expert, pair_row, pair_expert = self.route_native(routing_indices)
        weights = routing_weights.reshape(-1).contiguous()
        gate_up_bias, down_bias = self.gate_up_proj_bias.contiguous(), self.down_proj_bias.contiguous()

        # the kernels that fill the two padded buffers also leave their per-expert maxima (no amax pass of its own)
        amax = torch.zeros(2, self.num_experts, dtype=torch.float32, device=dev)
        padded = torch.empty(layout.capacity, self.hidden_size, dtype=dtype, device=dev)
        _native.check(lib.fos_experts_gather_rows(x.data_ptr(), code, x.stride(0), row_token.data_ptr(), padded.data_ptr(),
                                                  padded.stride(0), layout.capacity, self.hidden_size, row_expert.data_ptr(),
                                                  amax[0].data_ptr(), stream), "fos_experts_gather_rows")
        # padding rows of the two GEMM outputs are neither written nor read: no zero fill
        gu = torch.empty(layout.capacity, 2 * self.intermediate_size, dtype=dtype, device=dev)
        grouped_quantized_matmul(grouped_quantize(padded, layout, act_config, amax=amax[0]), gate_up, out_dtype=out_dtype, out=gu)
        gated = torch.empty(layout.capacity, self.intermediate_size, dtype=dtype, device=dev)
        _native.check(lib.fos_experts_glu(gu.data_ptr(), code, gu.stride(0), gate_up_bias.data_ptr(), row_expert.data_ptr(),
                                          gated.data_ptr(), gated.stride(0), layout.capacity, self.intermediate_size,
                                          float(self.alpha), float(self.limit), amax[1].data_ptr(), stream), "fos_experts_glu")
        y = torch.empty(layout.capacity, self.hidden_size, dtype=dtype, device=dev)
        grouped_quantized_matmul(grouped_quantize(gated, layout, act_config, amax=amax[1]), down, out_dtype=out_dtype, out=y)
        result = torch.empty(tokens, self.hidden_size, dtype=dtype, device=dev)
        _native.check(lib.fos_experts_combine(y.data_ptr(), code, y.stride(0), down_bias.data_ptr(), pair_row.data_ptr(),
                                              pair_expert.data_ptr(), weights.data_ptr(), top_k, result.data_ptr(),
                                              result.stride(0), tokens, self.hidden_size, stream), "fos_experts_combine")
        return result
