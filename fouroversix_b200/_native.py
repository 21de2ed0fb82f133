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
EXPERTS_ROUTE_WORKSPACE_INTS = 128                 # FOS_EXPERTS_ROUTE_WORKSPACE_INTS: per expert, for fos_experts_route
FOS_NVFP4, FOS_IF4, FOS_MXFP4 = 0, 1, 2
FOS_SF_ROWMAJOR, FOS_SF_TILED = 0, 1
FOS_QUANTIZE_EXACT_ONLY = 1
FOS_QUANTIZE_RHT = 2
FOS_QUANTIZE_NO_TMA = 4
FOS_QUANTIZE_GENERAL_KERNEL = 8
FOS_QUANTIZE_UNBIASED = 16
FOS_DEQUANT_VALUES_ONLY, FOS_DEQUANT_UNBIASED = 1, 2

_c_i64, _c_int, _c_ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p


class GemmOpts(ctypes.Structure):
    """fos_gemm_opts of include/fouroversix_b200.h: per-call kernel variant and CTA cap."""

    _fields_ = [("variant", ctypes.c_int32), ("max_ctas", ctypes.c_int32)]


def gemm_opts(variant: int = 0, max_ctas: int = 0):
    """A pointer argument for the *_ex GEMM entry points (None when everything is default)."""
    if not variant and not max_ctas:
        return None
    return ctypes.byref(GemmOpts(int(variant), int(max_ctas)))


# name -> (restype, argtypes); the list mirrors include/fouroversix_b200.h
SIGNATURES = {
    "fos_version": (_c_int, []),
    "fos_status_string": (ctypes.c_char_p, [_c_int]),
    "fos_last_cuda_error": (_c_int, []),
    "fos_quantize": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_int, _c_int,
                              _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr]),
    "fos_amax": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_quantize_stochastic": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_int, _c_int,
                                         _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, ctypes.c_uint64, _c_ptr]),
    "fos_pseudo_quantize": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr, _c_i64,
                                     _c_ptr, _c_int, _c_ptr]),
    "fos_dequantize": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_i64,
                                _c_ptr, _c_int, _c_i64, _c_ptr]),
    "fos_dequantize_ex": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_i64,
                                   _c_ptr, _c_int, _c_i64, _c_int, _c_int, _c_ptr]),
    "fos_gemm_alpha": (_c_int, [_c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr]),
    "fos_gemm_alpha_ex": (_c_int, [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr]),
    "fos_wait_failure_roles": (_c_int, [_c_ptr]),
    "fos_gemm_alpha_grouped": (_c_int, [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr]),
    "fos_gemm_nvfp4": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_i64, _c_i64,
                                _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_gemm_nvfp4_fused_a": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                        _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_quantize_grouped": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                                      _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr]),
    "fos_gemm_nvfp4_grouped": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                                        _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr]),
    "fos_linear_workspace_bytes": (_c_i64, [_c_i64, _c_i64]),
    "fos_linear_forward": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64,
                                    _c_ptr, _c_int, _c_i64, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr]),
    "fos_experts_workspace_bytes": (_c_i64, [_c_i64, _c_int, _c_int, _c_i64, _c_i64]),
    "fos_experts_forward": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_ptr, _c_int, _c_ptr, _c_int, _c_int,
                                     _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int,
                                     ctypes.c_float, ctypes.c_float, _c_ptr, _c_i64, _c_ptr, _c_i64, _c_ptr, _c_ptr]),
    "fos_experts_route": (_c_int, [_c_ptr, _c_int, _c_i64, _c_int, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                   _c_ptr, _c_ptr]),
    "fos_experts_gather_rows": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr]),
    "fos_experts_glu": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, ctypes.c_float,
                                 ctypes.c_float, _c_ptr, _c_ptr]),
    "fos_experts_combine": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_i64, _c_i64,
                                     _c_i64, _c_ptr]),
    "fos_gemm_mxfp4": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_i64, _c_i64,
                                _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_gemm_nvfp4_ex": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_i64, _c_i64,
                                   _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr]),
    "fos_gemm_mxfp4_ex": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_i64, _c_i64,
                                   _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr]),
    "fos_gemm_nvfp4_scatter": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_i64, _c_i64,
                                        _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "fos_allreduce_peer": (_c_int, [_c_ptr, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_ptr]),
    "fos_reduce_scatter_peer": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_i64, _c_int, _c_int, _c_ptr]),
    "fos_allgather_peer": (_c_int, [_c_ptr, _c_int, _c_i64, _c_i64, _c_ptr, _c_int, _c_ptr]),
    "fos_reduce_gather": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_i64, _c_int, _c_ptr]),
    "fos_gemm_if4_workspace_bytes": (_c_i64, [_c_i64, _c_i64, _c_i64]),
    "fos_gemm_if4": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                              _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_i64, _c_ptr, _c_ptr]),
    "fos_gemm_if4_static": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                                     _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
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


def wait_failure_site() -> int:
    """0, or the site of the first bounded device-side wait that ever gave up on the current device
    (quantize kernels 1-9, FP4 GEMM 100 + site, fp16 GEMM of the IF4 path 200 + site). Synchronises
    the device. Once it is non-zero, outputs of the kernels launched since are undefined."""
    site = ctypes.c_int32(0)
    check(lib().fos_wait_failure_site(ctypes.byref(site)), "fos_wait_failure_site")
    return int(site.value)


def wait_failure_roles() -> tuple[int, int, int]:
    """Bit masks of the wait sites that were blocked when a CTA gave up: (quantize kernels, FP4 GEMMs, IF4 GEMM)."""
    roles = (ctypes.c_uint32 * 3)()
    check(lib().fos_wait_failure_roles(roles), "fos_wait_failure_roles")
    return int(roles[0]), int(roles[1]), int(roles[2])


def raise_on_wait_failure() -> None:
    site = wait_failure_site()
    if site != 0:
        raise NativeLibraryError(f"a bounded device-side wait timed out (site {site}); results since then are undefined")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def elem_code(dtype: torch.dtype) -> int:
    try:
        return {torch.bfloat16: FOS_BF16, torch.float16: FOS_FP16, torch.float32: FOS_FP32}[dtype]
    except KeyError:
        raise ValueError(f"unsupported element type {dtype}") from None
