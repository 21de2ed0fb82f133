"""`FourOverSixLinear`: an `nn.Linear` whose matmuls run in FP4.

Forward:  y = q(x) @ q(W)^T (+ bias)                         one FP4 GEMM
Backward: dx = q(dy) @ q(W^T)^T ;  dW = q(dy^T) @ q(x^T)^T   two FP4 GEMMs
The transposed operands come from the quantize kernel's transposed mode, so no
high-precision transpose is materialised.

Interface, buffer names and buffer layouts follow the reference module
(src/fouroversix/model/modules/linear.py:40-453) so that state dicts interchange:
`quantized_weight_values` u8 [out, in/2], `quantized_weight_scale_factors` e4m3
[out*in/16], `quantized_weight_amax` f32 [1], `quantized_weight_metadata` i32 [6] =
(rows, cols, padded rows, padded cols, 1, scales-are-tiled).

Like the reference, the backward pass rotates both wgrad operands with the 16-point randomised
Hadamard transform before quantizing them (the rotation is orthogonal along the contracted
token axis, so it changes quantization error only) and rounds gradients as
`gradient_round_style` says (stochastic by default; the noise is seeded from torch's CPU
generator). Not implemented: `stochastic_unbiased` rounding and the Quartet-II backward.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from fouroversix_b200 import _native
from fouroversix_b200.matmul import quantized_matmul
from fouroversix_b200.quantize import QuantizedTensor, dequantize, quantize
from fouroversix_b200.utils import DataType, MatmulBackend, QuantizeBackend, RoundStyle

_TORCH_OUT = {DataType.bfloat16: torch.bfloat16, DataType.float16: torch.float16, DataType.float32: torch.float32}

from .config import ModuleQuantizationConfig
from .quantize import QuantizedModule


class FourOverSixLinearFunction(torch.autograd.Function):
    """Differentiable FP4 linear: apply(config, input, weight, bias)."""

    @staticmethod
    def forward(ctx, config: ModuleQuantizationConfig, input: torch.Tensor,
                weight: QuantizedTensor | nn.Parameter | torch.Tensor, bias: torch.Tensor | None = None):
        trainable = isinstance(weight, nn.Parameter)
        if trainable:
            ctx.config = config
            ctx.save_for_backward(input, weight, bias)

        x2d = input.reshape(-1, input.shape[-1])
        if config.disable_fprop_quantization:
            if isinstance(weight, QuantizedTensor):
                raise ValueError("disable_fprop_quantization needs the high-precision weight")
            out = x2d @ weight.T
            out_features = weight.shape[0]
        else:
            act_cfg = config.get_activation_config()
            if not isinstance(weight, QuantizedTensor):
                w = weight.data if trainable else weight
                weight = quantize(w, config.get_weight_config())
            if config.pseudo_quantize:
                # both operands fake-quantized, then a high-precision matmul
                out = quantize(x2d, act_cfg) @ weight.T
                out_features = weight.shape[0]
            else:
                out = quantized_matmul(x2d, weight, backend=config.matmul_backend, input_config=act_cfg,
                                       out_dtype=config.output_dtype)
                out_features = weight.original_shape[0]
        out = out.reshape(*input.shape[:-1], out_features)
        return out if bias is None else out + bias

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        input, weight, bias = ctx.saved_tensors
        cfg: ModuleQuantizationConfig = ctx.config
        if cfg.quartet_ii_dtype is not None:
            raise NotImplementedError("the Quartet-II backward pass is not implemented")
        # settings of the reference's backward pass (src/fouroversix/model/modules/linear.py:213-229, 258-268)
        # that this layer does not implement are refused rather than silently ignored
        if getattr(cfg, "wgrad_nvint4", False):
            raise NotImplementedError("wgrad_nvint4 is not implemented")
        if isinstance(cfg.disable_dgrad_quantization, str):
            raise NotImplementedError(
                f"disable_dgrad_quantization={cfg.disable_dgrad_quantization!r} is not implemented (True / False are)")

        dy = grad_output.reshape(-1, grad_output.shape[-1])     # [tokens, out]
        x = input.reshape(-1, input.shape[-1])                   # [tokens, in]
        w = weight.data                                          # [out, in]

        # dgrad: dx[tokens, in] = dy @ W = q(dy) @ q(W^T)^T
        if cfg.disable_dgrad_quantization:
            dx = dy @ w
        elif cfg.pseudo_quantize:
            dx = quantize(dy, cfg.get_gradient_config()) @ quantize(w, cfg.get_weight_config(transpose=True)).T
        else:
            dx = quantized_matmul(dy, w, backend=cfg.matmul_backend, input_config=cfg.get_gradient_config(),
                                  other_config=cfg.get_weight_config(transpose=True), out_dtype=cfg.output_dtype)
        dx = dx.reshape(*grad_output.shape[:-1], w.shape[1])

        # wgrad: dW[out, in] = dy^T @ x = q(rot(dy^T)) @ q(rot(x^T))^T, rotation along the token axis
        # (src/fouroversix/model/modules/linear.py:245-256)
        if cfg.disable_wgrad_quantization:
            dw = dy.T @ x
        elif cfg.pseudo_quantize:
            dw = quantize(dy, cfg.get_gradient_config(rht=True, transpose=True)) @ \
                quantize(x, cfg.get_activation_config(rht=True, transpose=True)).T
        else:
            dw = quantized_matmul(dy, x, backend=cfg.matmul_backend,
                                  input_config=cfg.get_gradient_config(rht=True, transpose=True),
                                  other_config=cfg.get_activation_config(rht=True, transpose=True),
                                  out_dtype=cfg.output_dtype)

        db = dy.sum(0) if bias is not None and ctx.needs_input_grad[3] else None
        return None, dx, dw.to(w.dtype), db


@QuantizedModule.register(nn.Linear)
class FourOverSixLinear(nn.Linear):
    """Drop-in replacement for `nn.Linear` built from an existing layer and a config."""

    def __init__(self, module: nn.Linear, config: ModuleQuantizationConfig) -> None:
        super().__init__(module.in_features, module.out_features, module.bias is not None,
                         device="meta", dtype=module.weight.dtype)
        self.weight = module.weight
        self.bias = module.bias
        self.config = config
        if not config.keep_master_weights:
            dev = module.weight.device
            wd = config.weight_dtype
            packed = wd.quantized_value_type.packing_factor

            def buf(name: str, tensor: torch.Tensor) -> None:
                self.register_buffer(name, nn.Parameter(tensor, requires_grad=False))

            buf("quantized_weight_values",
                torch.zeros(self.out_features, self.in_features // packed, dtype=torch.uint8, device=dev))
            buf("quantized_weight_scale_factors",
                torch.zeros(self.out_features * self.in_features // wd.block_size,
                            dtype=wd.scale_type.torch_dtype, device=dev))
            buf("quantized_weight_amax", torch.zeros(1, dtype=torch.float32, device=dev))
            buf("quantized_weight_metadata", torch.zeros(6, dtype=torch.int32, device=dev))

    @property
    def parameters_to_quantize(self) -> tuple[str, ...]:
        """High-precision parameters that a loader should quantize and then drop."""
        return ("weight",)

    def get_element_size(self, parameter_name: str) -> float:
        """Bytes per element of a parameter once quantized (packed values: 0.5; a whole
        quantized weight: 8 bytes of values + 1 scale byte per 16 elements)."""
        special = {"quantized_weight_values": 0.5, "weight": 9 / 16}
        if parameter_name in special:
            return special[parameter_name]
        return getattr(self, parameter_name).element_size()

    def get_quantized_parameters(self, parameter_name: str, parameter: torch.Tensor) -> dict[str, Any]:
        """Quantize a high-precision weight (on the GPU) into the four packed buffers."""
        if parameter_name != "weight":
            raise ValueError(f"Unsupported high-precision parameter: {parameter_name}")
        q = quantize(parameter, self.config.get_weight_config())
        meta = [q.original_shape[0], q.original_shape[1], q.padded_shape[0], q.padded_shape[1], 1,
                int(q.scale_factors_are_in_blackwell_layout)]
        return {
            "quantized_weight_values": q.values,
            "quantized_weight_scale_factors": q.scale_factors,
            "quantized_weight_amax": q.amax,
            "quantized_weight_metadata": torch.tensor(meta, dtype=torch.int32),
        }

    def quantize_weight_(self) -> "FourOverSixLinear":
        """Post-training quantization in place: fill the packed buffers from `weight` and
        drop the high-precision copy.  (The reference leaves this step to its model
        loaders; here it is one call.)"""
        if self.config.keep_master_weights:
            raise ValueError("quantize_weight_ is for keep_master_weights=False modules")
        params = self.get_quantized_parameters("weight", self.weight.data)
        for name, value in params.items():
            setattr(self, name, nn.Parameter(value.to(self.weight.device), requires_grad=False))
        self.weight = None
        self.__dict__.pop("_quantized_weight", None)
        return self

    def quantized_weight(self) -> QuantizedTensor | nn.Parameter:
        """The weight operand of the forward GEMM: the master weight when it is kept,
        else a `QuantizedTensor` view of the packed buffers (built once and cached)."""
        if self.config.keep_master_weights:
            return self.weight
        cached = self.__dict__.get("_quantized_weight")
        if cached is None:
            meta = self.quantized_weight_metadata.data.tolist()
            if meta[0] == 0:
                raise RuntimeError("the packed weight buffers are empty: load a quantized state dict or call "
                                   "quantize_weight_() first")
            cached = QuantizedTensor(
                self.quantized_weight_values.data, self.quantized_weight_scale_factors.data,
                self.quantized_weight_amax.data, self.config.weight_dtype, tuple(meta[0:2]),
                self.config.weight_scale_rule, self.config.weight_round_style, tuple(meta[2:4]),
                scale_factors_are_in_blackwell_layout=meta[5] == 1)
            self.__dict__["_quantized_weight"] = cached
        return cached

    def dequantized_weight(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """High-precision copy of the stored weight (debugging / export)."""
        w = self.quantized_weight()
        return dequantize(w, dtype) if isinstance(w, QuantizedTensor) else w.data.to(dtype)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self._one_call_forward_applies(input):
            return self._forward_one_call(input)
        return FourOverSixLinearFunction.apply(self.config, input, self.quantized_weight(), self.bias)

    def _one_call_forward_applies(self, input: torch.Tensor) -> bool:
        """Inference on a packed NVFP4 weight with the plain activation settings (NVFP4, 1-D blocks, round to
        nearest): the case `fos_linear_forward` covers. Everything else (training, master weights, other formats,
        fake quantization) goes through the autograd function."""
        cfg = self.config
        if (cfg.keep_master_weights or cfg.disable_fprop_quantization or cfg.pseudo_quantize
                or cfg.activation_dtype != DataType.nvfp4 or cfg.activation_round_style != RoundStyle.nearest
                or cfg.matmul_backend not in (None, MatmulBackend.cutlass)
                or cfg.quantize_backend not in (None, QuantizeBackend.cuda)):
            return False
        if (torch.is_grad_enabled() and input.requires_grad) or not input.is_cuda:
            return False
        if input.dtype not in (torch.bfloat16, torch.float16) or input.shape[-1] != self.in_features or input.numel() == 0:
            return False
        w = self.quantized_weight()
        return (isinstance(w, QuantizedTensor) and w.dtype == DataType.nvfp4 and w.scale_factors_are_in_blackwell_layout
                and w.round_style != RoundStyle.stochastic_unbiased and w.values.is_contiguous()
                and w.scale_factors.is_contiguous())

    def _forward_one_call(self, input: torch.Tensor) -> torch.Tensor:
        """`fos_linear_forward`: amax pass, activation quantization, alpha and the GEMM enqueued by one host call
        (the bits of `quantized_matmul(input, weight)`; at decode sizes the call-by-call form is bound by the
        interpreter)."""
        w = self.quantized_weight()
        x = input.reshape(-1, self.in_features)
        if x.stride(-1) != 1:
            x = x.contiguous()
        dev, rows = x.device, x.shape[0]
        out_dtype = _TORCH_OUT[DataType(self.config.output_dtype)]
        lib = _native.lib()
        need = lib.fos_linear_workspace_bytes(rows, self.in_features)
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        out = torch.empty(rows, self.out_features, dtype=out_dtype, device=dev)
        def launch() -> None:
            _native.check(lib.fos_linear_forward(
                x.data_ptr(), _native.elem_code(x.dtype), rows, self.in_features, x.stride(0),
                self.config.activation_scale_rule.cuda_id, w.values.data_ptr(), w.scale_factors.data_ptr(),
                w.amax.data_ptr(), w.scale_rule.cuda_id, self.out_features, out.data_ptr(), _native.elem_code(out_dtype),
                out.stride(0), workspace.data_ptr(), need, None, 0, _native.stream_ptr(dev)), "fos_linear_forward")

        if dev.index is None or dev.index == torch.cuda.current_device():
            launch()                                  # (entering a device context costs microseconds a decode step feels)
        else:
            with torch.cuda.device(dev):
                launch()
        out = out.reshape(*input.shape[:-1], self.out_features)
        return out if self.bias is None else out + self.bias
