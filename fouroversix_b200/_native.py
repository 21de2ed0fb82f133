"""ctypes binding of libfouroversix_b200.so (the C ABI declared in include/fouroversix_b200.h).

There is no fallback: if the shared library is missing, loading raises, and every GPU
entry point of the package fails with that error.  Build it with
`python -m fouroversix_b200.build`.
"""

from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libfouroversix_b200.so"
_lib: ctypes.CDLL | None = None

FOS_BF16, FOS_FP16, FOS_FP32 = 0, 1, 2
FOS_NVFP4, FOS_IF4, FOS_MXFP4 = 0, 1, 2
FOS_SF_ROWMAJOR, FOS_SF_TILED = 0, 1
FOS_QUANTIZE_EXACT_ONLY = 1
FOS_QUANTIZE_RHT = 2
FOS_OPT_GEMM_MAX_CTAS = 4

_c_i64, _c_int, _c_ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p

# name -> (restype, argtypes); the list mirrors include/fouroversix_b200.h
SIGNATURES = {
    "fos_version": (_c_int, []),
    "fos_status_string": (ctypes.c_char_p, [_c_int]),
    "fos_last_cuda_error": (_c_int, []),
    "fos_quantize": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_int, _c_int,
                              _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr]),
    "fos_quantize_stochastic": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_int, _c_int,
                                         _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, ctypes.c_uint64, _c_ptr]),
    "fos_pseudo_quantize": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr, _c_i64,
                                     _c_ptr, _c_int, _c_ptr]),
    "fos_dequantize": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_i64,
                                _c_ptr, _c_int, _c_i64, _c_ptr]),
    "fos_gemm_alpha": (_c_int, [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr]),
    "fos_gemm_nvfp4": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_i64, _c_i64,
                                _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_gemm_mxfp4": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_i64, _c_i64,
                                _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_gemm_nvfp4_scatter": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64,
                                        _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_allreduce_peer": (_c_int, [_c_ptr, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_ptr]),
    "fos_reduce_gather": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_ptr]),
    "fos_gemm_if4_workspace_bytes": (_c_i64, [_c_i64, _c_i64, _c_i64]),
    "fos_gemm_if4": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                              _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_i64, _c_ptr, _c_ptr]),
    "fos_gemm_if4_static": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                                     _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_set_option": (_c_int, [_c_int, _c_int]),
    "fos_wait_failure_site": (_c_int, [_c_ptr]),
}


class NativeLibraryError(RuntimeError):
    """The CUDA extension is missing or a call into it failed."""


def library_path() -> Path:
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise NativeLibraryError(
                f"{_LIB_PATH} not found: the CUDA extension has not been built "
                "(python -m fouroversix_b200.build); there is no fallback path")
        loaded = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(loaded, name, None)
            if fn is None:
                continue  # reported by exported_symbols(); callers of a missing symbol fail loudly
            fn.restype, fn.argtypes = res, args
        _lib = loaded
    return _lib


def exported_symbols() -> dict[str, bool]:
    loaded = lib()
    return {name: hasattr(loaded, name) for name in SIGNATURES}


def check(status: int, what: str) -> None:
    if status == 0:
        return
    l = lib()
    msg = l.fos_status_string(status).decode()
    if status == -4:
        msg += f" (cudaError {l.fos_last_cuda_error()})"
    exc = ValueError if status in (-1, -2, -3, -7) else NativeLibraryError
    raise exc(f"{what}: {msg}")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def elem_code(dtype: torch.dtype) -> int:
    try:
        return {torch.bfloat16: FOS_BF16, torch.float16: FOS_FP16, torch.float32: FOS_FP32}[dtype]
    except KeyError:
        raise ValueError(f"unsupported element type {dtype}") from None
