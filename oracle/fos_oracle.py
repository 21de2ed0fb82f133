"""ctypes front end of the CPU oracle (oracle/fos_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped package never imports this module.

The functions take and return CPU torch tensors so that a test can feed the same
bits to the oracle and to the CUDA kernels.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB: ctypes.CDLL | None = None

FORMATS = {"nvfp4": 0, "if4": 1, "mxfp4": 2}
# Same numbering as the reference's ScaleRule.cuda_id (src/fouroversix/utils.py:271-280).
RULES = {"static_6": 0, "static_4": 1, "mae": 2, "mse": 3, "abs_max": 4}
OUT_TYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def lib() -> ctypes.CDLL:
    """Load oracle/libfos_oracle.so, compiling it first when gcc is at hand."""
    global _LIB
    if _LIB is None:
        so = _HERE / "libfos_oracle.so"
        if not so.exists():
            import importlib.util

            spec = importlib.util.spec_from_file_location("_fos_oracle_build", _HERE / "build.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build()
        _LIB = ctypes.CDLL(str(so))
        _LIB.fos_oracle_alpha.restype = ctypes.c_float
        _LIB.fos_oracle_alpha.argtypes = [ctypes.c_float, ctypes.c_int, ctypes.c_int] * 2
    return _LIB


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _name(v) -> str:
    return getattr(v, "value", v)


@dataclass
class OracleQuantized:
    """What the reference's PyTorch backend returns for one tensor, plus diagnostics."""

    values: torch.Tensor          # uint8 [Rp, Cp/2]
    scale_factors: torch.Tensor   # uint8 [Rp*Cp/16] ([Rp*Cp/32] for mxfp4); 128x4-tiled for nvfp4 / mxfp4, row-major for if4
    amax: torch.Tensor            # float32 [1]
    choice: torch.Tensor          # uint8 [Rp, Cp/16]: 1 where "4" (nvfp4) or "int" (if4) won
    worst_scaled: float           # max |x / scale| over all candidates
    dtype: str
    scale_rule: str
    original_shape: tuple[int, int]
    padded_shape: tuple[int, int]
    tiled: bool


def rht(x: torch.Tensor, *, transpose: bool = False) -> torch.Tensor:
    """The reference's 16-point random Hadamard transform of x (of x^T when `transpose`), in x's dtype."""
    assert x.device.type == "cpu" and x.ndim == 2 and x.stride(1) == 1
    assert x.dtype in (torch.bfloat16, torch.float16)
    R, C = x.shape
    out = torch.empty((C, R) if transpose else (R, C), dtype=x.dtype)
    rc = lib().fos_oracle_rht(_ptr(x), ctypes.c_int(x.dtype == torch.float16), ctypes.c_int64(R), ctypes.c_int64(C),
                              ctypes.c_int64(x.stride(0)), ctypes.c_int(transpose), _ptr(out))
    if rc != 0:
        raise ValueError("the rotated axis must be a multiple of 16")
    return out


def quantize(
    x: torch.Tensor,
    *,
    dtype="nvfp4",
    scale_rule="mse",
    block_scale_2d: bool = False,
    transpose: bool = False,
    amax: torch.Tensor | None = None,
    rht: bool = False,
) -> OracleQuantized:
    if rht:
        # rotate first (after the transposition, as the reference does), then quantize as usual
        return quantize(globals()["rht"](x, transpose=transpose), dtype=dtype, scale_rule=scale_rule,
                        block_scale_2d=block_scale_2d, transpose=False, amax=amax)
    dtype, scale_rule = _name(dtype), _name(scale_rule)
    assert x.device.type == "cpu" and x.ndim == 2 and x.stride(1) == 1
    assert x.dtype in (torch.bfloat16, torch.float16)
    R, C = x.shape
    Ro, Co = (C, R) if transpose else (R, C)
    bw = 32 if dtype == "mxfp4" else 16                      # block width
    Rp, Cp = -(-Ro // 128) * 128, -(-Co // (4 * bw)) * (4 * bw)
    tiled = dtype != "if4"
    values = torch.empty(Rp, Cp // 2, dtype=torch.uint8)
    sf = torch.empty(Rp * Cp // bw, dtype=torch.uint8)
    amax_out = torch.empty(1, dtype=torch.float32)
    choice = torch.empty(Rp, Cp // bw, dtype=torch.uint8)
    worst = ctypes.c_float(0.0)
    amax_in = None if amax is None else amax.detach().to(torch.float32).reshape(1).contiguous()
    rc = lib().fos_oracle_quantize(
        _ptr(x), ctypes.c_int(x.dtype == torch.float16),
        ctypes.c_int64(R), ctypes.c_int64(C), ctypes.c_int64(x.stride(0)),
        ctypes.c_int(FORMATS[dtype]), ctypes.c_int(RULES[scale_rule]),
        ctypes.c_int(block_scale_2d), ctypes.c_int(transpose), ctypes.c_int(tiled),
        _ptr(amax_in), _ptr(values), _ptr(sf), _ptr(amax_out), _ptr(choice), ctypes.byref(worst),
    )
    if rc != 0:
        raise ValueError(f"oracle rejected dtype={dtype} scale_rule={scale_rule}")
    return OracleQuantized(values, sf, amax_out, choice, worst.value, dtype, scale_rule,
                           (Ro, Co), (Rp, Cp), tiled)


def dequantize(q: OracleQuantized, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    return dequantize_raw(q.values, q.scale_factors, q.amax, q.dtype, q.scale_rule,
                          q.original_shape, dtype, tiled=q.tiled)


def dequantize_raw(values, scale_factors, amax, dtype, scale_rule, original_shape,
                   out_dtype=torch.bfloat16, *, tiled: bool | None = None) -> torch.Tensor:
    dtype, scale_rule = _name(dtype), _name(scale_rule)
    tiled = (dtype == "nvfp4") if tiled is None else tiled
    values = values.contiguous()
    sf = scale_factors.contiguous().view(torch.uint8).flatten()
    Rp, Cp = values.shape[0], values.shape[1] * 2
    R, C = original_shape
    out = torch.empty(R, C, dtype=out_dtype)
    amax = amax.detach().to(torch.float32).reshape(1).contiguous()
    lib().fos_oracle_dequantize(
        _ptr(values), _ptr(sf), _ptr(amax), ctypes.c_int(FORMATS[dtype]),
        ctypes.c_int(RULES[scale_rule]), ctypes.c_int(tiled),
        ctypes.c_int64(Rp), ctypes.c_int64(Cp), ctypes.c_int64(R), ctypes.c_int64(C),
        ctypes.c_int(OUT_TYPES[out_dtype]), _ptr(out),
    )
    return out


def alpha(qa: OracleQuantized, qb: OracleQuantized) -> float:
    return float(lib().fos_oracle_alpha(
        ctypes.c_float(qa.amax.item()), FORMATS[qa.dtype], RULES[qa.scale_rule],
        ctypes.c_float(qb.amax.item()), FORMATS[qb.dtype], RULES[qb.scale_rule]))


def matmul(qa: OracleQuantized, qb: OracleQuantized, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """deq32(a) @ deq32(b).T with fp32 accumulation, cast to out_dtype (all in C)."""
    M, K = qa.original_shape
    N, Kb = qb.original_shape
    assert K == Kb and qa.padded_shape[1] == qb.padded_shape[1]
    out = torch.empty(M, N, dtype=out_dtype)
    rc = lib().fos_oracle_matmul(
        _ptr(qa.values), _ptr(qa.scale_factors), _ptr(qa.amax), ctypes.c_int(FORMATS[qa.dtype]),
        ctypes.c_int(RULES[qa.scale_rule]), ctypes.c_int(qa.tiled), ctypes.c_int64(qa.padded_shape[0]),
        _ptr(qb.values), _ptr(qb.scale_factors), _ptr(qb.amax), ctypes.c_int(FORMATS[qb.dtype]),
        ctypes.c_int(RULES[qb.scale_rule]), ctypes.c_int(qb.tiled), ctypes.c_int64(qb.padded_shape[0]),
        ctypes.c_int64(qa.padded_shape[1]), ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K),
        ctypes.c_int(OUT_TYPES[out_dtype]), _ptr(out),
    )
    assert rc == 0
    return out


def num_threads() -> int:
    return int(lib().fos_oracle_num_threads())


def set_num_threads(n: int) -> None:
    """Use `n` OpenMP threads from now on (launchers like torchrun export OMP_NUM_THREADS=1)."""
    lib().fos_oracle_set_num_threads(ctypes.c_int(int(n)))
