"""The one matmul back end: the hand-written tcgen05 block-scaled FP4 GEMM.

It fills the role of the reference's CUTLASS back end
(src/fouroversix/matmul/cutlass/backend.py:10-155; shape check from
src/fouroversix/matmul/backend.py:32-38): `input @ other.T` for two NVFP4
`QuantizedTensor`s with `alpha = amax_a * amax_b / (divisor_a * divisor_b)` applied in
the epilogue.  alpha is computed on the device, so the call never synchronises.
"""

from __future__ import annotations

import torch

from fouroversix_b200 import _native
from fouroversix_b200.quantize import QuantizedTensor
from fouroversix_b200.quantize.backend import B200QuantizeBackend
from fouroversix_b200.utils import DataType, RoundStyle

_OUT = {DataType.bfloat16: torch.bfloat16, DataType.float16: torch.float16, DataType.float32: torch.float32}
_FORMATS = {DataType.nvfp4: _native.FOS_NVFP4, DataType.if4: _native.FOS_IF4, DataType.mxfp4: _native.FOS_MXFP4}


def _layout(q: QuantizedTensor) -> int:
    return _native.FOS_SF_TILED if q.scale_factors_are_in_blackwell_layout else _native.FOS_SF_ROWMAJOR


class B200MatmulBackend:
    """FP4 x FP4 -> bf16 / fp16 / fp32 on the 5th-generation tensor cores: block-scaled
    kind::mxf4nvf4 MMAs for NVFP4 operands, kind::mxf4 MMAs for MXFP4 operands (alpha = 1, as in
    src/fouroversix/matmul/cutlass/backend.py:79-84), expand-to-fp16 + kind::f16 MMAs for IF4."""

    @classmethod
    def is_available(cls) -> bool:
        return B200QuantizeBackend.is_available()

    @classmethod
    def unsupported_reason(cls, input: QuantizedTensor, other: QuantizedTensor, *, out_dtype: DataType) -> str | None:
        if input.original_shape[1] != other.original_shape[1]:
            # same wording as the reference's shape check
            raise ValueError(
                "The first input must be in row-major layout, the second input must be"
                "in column-major layout, and both inputs must have the same inner "
                "dimension")
        if input.dtype not in _FORMATS or other.dtype not in _FORMATS:
            return "operands must be nvfp4, if4 or mxfp4"
        if (input.dtype == DataType.mxfp4) != (other.dtype == DataType.mxfp4):
            return "an mxfp4 operand needs an mxfp4 partner"
        if input.dtype == DataType.mxfp4 and not (input.scale_factors_are_in_blackwell_layout
                                                  and other.scale_factors_are_in_blackwell_layout):
            return "mxfp4 operands need their scales in the tile layout"
        if input.device.type != "cuda" or other.device != input.device:
            return "both operands must live on the same CUDA device"
        if DataType(out_dtype) not in _OUT:
            return f"output type {out_dtype} is not supported"
        return None

    @classmethod
    def is_supported(cls, input: QuantizedTensor, other: QuantizedTensor, *, out_dtype: DataType) -> bool:
        return cls.unsupported_reason(input, other, out_dtype=out_dtype) is None and cls.is_available()

    @classmethod
    def quantized_matmul(cls, input: QuantizedTensor, other: QuantizedTensor, *, out_dtype: DataType,
                         out: torch.Tensor | None = None, check_status: bool = False, variant: int = 0,
                         max_ctas: int = 0) -> torch.Tensor:
        """`input @ other.T`, cropped to (input rows, other rows).  `check_status` reads the
        kernel's device status word back (one synchronisation) and raises on a timeout; without it a
        wait that gives up leaves its site in the library's sticky word (`_native.raise_on_wait_failure`).
        `variant` / `max_ctas` are the per-call options of the FP4 kernels (fos_gemm_opts): which
        kernel, and how many CTAs at most (to leave SMs to a collective running beside the GEMM)."""
        reason = cls.unsupported_reason(input, other, out_dtype=out_dtype)
        if reason is not None:
            raise ValueError(f"B200 matmul: {reason}")
        dev = input.device
        m, n = input.original_shape[0], other.original_shape[0]
        m_p, k_p = input.padded_shape
        n_p = other.padded_shape[0]
        if other.padded_shape[1] != k_p:
            raise ValueError("B200 matmul: operands are padded to different inner dimensions")
        torch_out = _OUT[DataType(out_dtype)]
        if out is None:
            out = torch.empty(m, n, dtype=torch_out, device=dev)
        elif out.shape != (m, n) or out.dtype != torch_out or out.stride(1) != 1:
            raise ValueError("B200 matmul: `out` has the wrong shape, dtype or layout")
        alpha = torch.empty(1, dtype=torch.float32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev) if check_status else None
        a_vals, b_vals = input.values.contiguous(), other.values.contiguous()
        a_sf, b_sf = input.scale_factors.contiguous(), other.scale_factors.contiguous()
        fa, fb = _FORMATS[input.dtype], _FORMATS[other.dtype]
        # block-scaled FP4 tensor cores when both operands are NVFP4 in the tile layout; otherwise
        # (IF4, or row-major scales) the fp16 path, which needs a scratch buffer for the expanded operands
        native_fp4 = (fa == fb == _native.FOS_NVFP4 and _layout(input) == _layout(other) == _native.FOS_SF_TILED)
        with torch.cuda.device(dev):
            lib, stream = _native.lib(), _native.stream_ptr(dev)
            status_ptr = 0 if status is None else status.data_ptr()
            opts = _native.gemm_opts(variant, max_ctas)
            if fa == _native.FOS_MXFP4:
                alpha.fill_(1.0)
                _native.check(lib.fos_gemm_mxfp4_ex(
                    a_vals.data_ptr(), a_sf.data_ptr(), b_vals.data_ptr(), b_sf.data_ptr(), alpha.data_ptr(),
                    out.data_ptr(), _native.elem_code(torch_out), m_p, n_p, k_p, m, n, out.stride(0),
                    opts, status_ptr, stream), "fos_gemm_mxfp4")
                if status is not None and int(status.item()) != 0:
                    raise _native.NativeLibraryError(
                        f"fos_gemm_mxfp4: a bounded device-side wait timed out (site {int(status.item())})")
                return out
            _native.check(lib.fos_gemm_alpha_ex(
                input.amax.data_ptr(), fa, input.scale_rule.cuda_id, int(input.round_style == RoundStyle.stochastic_unbiased),
                other.amax.data_ptr(), fb, other.scale_rule.cuda_id, int(other.round_style == RoundStyle.stochastic_unbiased),
                alpha.data_ptr(), stream), "fos_gemm_alpha")
            if native_fp4:
                _native.check(lib.fos_gemm_nvfp4_ex(
                    a_vals.data_ptr(), a_sf.data_ptr(), b_vals.data_ptr(), b_sf.data_ptr(), alpha.data_ptr(),
                    out.data_ptr(), _native.elem_code(torch_out), m_p, n_p, k_p, m, n, out.stride(0),
                    opts, status_ptr, stream), "fos_gemm_nvfp4")
            else:
                nbytes = int(lib.fos_gemm_if4_workspace_bytes(m_p, n_p, k_p))
                workspace = torch.empty(nbytes, dtype=torch.uint8, device=dev)
                _native.check(lib.fos_gemm_if4(
                    a_vals.data_ptr(), a_sf.data_ptr(), fa, _layout(input),
                    b_vals.data_ptr(), b_sf.data_ptr(), fb, _layout(other), alpha.data_ptr(),
                    out.data_ptr(), _native.elem_code(torch_out), m_p, n_p, k_p, m, n, out.stride(0),
                    workspace.data_ptr(), nbytes, status_ptr, stream), "fos_gemm_if4")
        if status is not None and int(status.item()) != 0:
            raise _native.NativeLibraryError(
                f"fos_gemm_nvfp4: a bounded device-side wait timed out (site {int(status.item())})")
        return out

    @classmethod
    def fused_quantize_matmul(cls, x: torch.Tensor, other: QuantizedTensor, config, *, out_dtype: DataType,
                              amax: torch.Tensor | None = None, out: torch.Tensor | None = None,
                              check_status: bool = False) -> torch.Tensor:
        """`quantize(x, config) @ other.T` with the quantization of x done inside the GEMM
        (fos_gemm_nvfp4_fused_a): the packed activation is never written to memory. For NVFP4 with a static
        scale rule, 1-D blocks, round to nearest; bit-identical to the two calls it replaces (the un-fused pair
        of src/fouroversix/matmul/frontend.py:95-102). `amax` (max |x|, a CUDA fp32 tensor) is computed with
        one pass over x when it is not given. Raises ValueError for what the fused kernel does not take: the
        caller then quantizes first."""
        from fouroversix_b200.utils import RoundStyle, ScaleRule

        if (DataType(config.dtype) != DataType.nvfp4 or ScaleRule(config.scale_rule) not in (ScaleRule.static_6, ScaleRule.static_4)
                or config.block_scale_2d or config.transpose or config.rht or RoundStyle(config.round_style) != RoundStyle.nearest):
            raise ValueError("B200 fused matmul: the activation must be NVFP4 with static_6 / static_4, 1-D blocks, "
                             "round to nearest (the 4/6 rules are not fused)")
        if other.dtype != DataType.nvfp4 or not other.scale_factors_are_in_blackwell_layout:
            raise ValueError("B200 fused matmul: the second operand must be NVFP4 with tiled scales")
        if x.ndim != 2 or x.device.type != "cuda" or x.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("B200 fused matmul: x must be a 2-D bfloat16 / float16 CUDA tensor")
        if x.stride(1) != 1:
            x = x.contiguous()
        m, k = x.shape
        n = other.original_shape[0]
        n_p, k_p = other.padded_shape
        if other.original_shape[1] != k:
            raise ValueError("The first input must be in row-major layout, the second input must be"
                             "in column-major layout, and both inputs must have the same inner "
                             "dimension")
        if k % 64 or k_p != k or x.data_ptr() % 32 or (x.stride(0) * 2) % 32:
            raise ValueError("B200 fused matmul: K must be a multiple of 64 and x 32-byte aligned (base and row stride)")
        dev = x.device
        torch_out = _OUT[DataType(out_dtype)]
        if out is None:
            out = torch.empty(m, n, dtype=torch_out, device=dev)
        elif out.shape != (m, n) or out.dtype != torch_out or out.stride(1) != 1:
            raise ValueError("B200 matmul: `out` has the wrong shape, dtype or layout")
        if amax is None:
            amax = B200QuantizeBackend.amax(x)
        amax = amax.detach().reshape(1).to(device=dev, dtype=torch.float32)
        alpha = torch.empty(1, dtype=torch.float32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev) if check_status else None
        rule = ScaleRule(config.scale_rule).cuda_id
        with torch.cuda.device(dev):
            lib, stream = _native.lib(), _native.stream_ptr(dev)
            _native.check(lib.fos_gemm_alpha(amax.data_ptr(), _native.FOS_NVFP4, rule, other.amax.data_ptr(), _native.FOS_NVFP4,
                                             other.scale_rule.cuda_id, alpha.data_ptr(), stream), "fos_gemm_alpha")
            _native.check(lib.fos_gemm_nvfp4_fused_a(
                x.data_ptr(), _native.elem_code(x.dtype), x.stride(0), amax.data_ptr(), rule,
                other.values.contiguous().data_ptr(), other.scale_factors.contiguous().data_ptr(), alpha.data_ptr(),
                out.data_ptr(), _native.elem_code(torch_out), m, n_p, k, n, out.stride(0),
                0 if status is None else status.data_ptr(), stream), "fos_gemm_nvfp4_fused_a")
        if status is not None and int(status.item()) != 0:
            raise _native.NativeLibraryError(
                f"fos_gemm_nvfp4_fused_a: a bounded device-side wait timed out (site {int(status.item())})")
        return out

    @classmethod
    def quantized_matmul_scatter(cls, input: QuantizedTensor, other: QuantizedTensor, *, out_dtype: DataType,
                                 d_peers, world: int, rank: int) -> None:
        """First half of a row-parallel layer's exchange: this rank's partial product `input @ other.T`, each
        tile stored as it completes into plane `rank` of the staging buffer of the rank that owns its rows
        (fos_gemm_nvfp4_scatter). `d_peers` is a ctypes array of `world` device pointers to the staging
        buffers [world][rows / world][n] of all ranks as mapped into this process."""
        reason = cls.unsupported_reason(input, other, out_dtype=out_dtype)
        if reason is not None:
            raise ValueError(f"B200 matmul: {reason}")
        if not (input.dtype == other.dtype == DataType.nvfp4 and _layout(input) == _layout(other) == _native.FOS_SF_TILED):
            raise ValueError("B200 matmul: the scatter epilogue needs two NVFP4 operands with tiled scales")
        dev = input.device
        m, n = input.original_shape[0], other.original_shape[0]
        m_p, k_p = input.padded_shape
        n_p = other.padded_shape[0]
        if other.padded_shape[1] != k_p:
            raise ValueError("B200 matmul: operands are padded to different inner dimensions")
        torch_out = _OUT[DataType(out_dtype)]
        alpha = torch.empty(1, dtype=torch.float32, device=dev)
        a_vals, b_vals = input.values.contiguous(), other.values.contiguous()
        a_sf, b_sf = input.scale_factors.contiguous(), other.scale_factors.contiguous()
        with torch.cuda.device(dev):
            lib, stream = _native.lib(), _native.stream_ptr(dev)
            _native.check(lib.fos_gemm_alpha(
                input.amax.data_ptr(), _native.FOS_NVFP4, input.scale_rule.cuda_id,
                other.amax.data_ptr(), _native.FOS_NVFP4, other.scale_rule.cuda_id, alpha.data_ptr(), stream), "fos_gemm_alpha")
            _native.check(lib.fos_gemm_nvfp4_scatter(
                a_vals.data_ptr(), a_sf.data_ptr(), b_vals.data_ptr(), b_sf.data_ptr(), alpha.data_ptr(),
                d_peers, world, rank, _native.elem_code(torch_out), m_p, n_p, k_p, m, n, n, 0, stream),
                "fos_gemm_nvfp4_scatter")

