"""The IF4 GEMM entry point that takes no workspace (`fos_gemm_if4_static`).

Some callers cannot give the library scratch memory: they run where allocating device memory
is not allowed (a plug-in hook of another framework that may launch kernels but must leave the
allocator alone, a memory pool that has already been handed out completely). For them the library keeps a fixed 32 MiB buffer inside
its own image. This test calls that entry point through the C ABI, twice in a row on different
data, and requires bit-identical results to `fos_gemm_if4` with a caller-provided workspace
(the same kernels run in both, so there is no tolerance to apply); it measures that the call
leaves the device's free memory and torch's allocator untouched; and it checks that a problem
beyond the fixed buffer is refused with FOS_ERR_TOO_LARGE.

The file name makes pytest collect it last, so a run that stops at the first failure has
already executed every other test.
"""

from __future__ import annotations

import pytest
import torch

import fouroversix_b200 as fos
from fouroversix_b200 import _native

pytestmark = pytest.mark.gpu

DEV = "cuda"
FOS_ERR_TOO_LARGE = -7


def _operands(seed: int, m: int, n: int, k: int):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().to(DEV)
    cfg = fos.QuantizationConfig(dtype="if4")
    return fos.quantize(x, cfg), fos.quantize(w, cfg)


def _call(static: bool, qa, qb, out, alpha, workspace=None) -> int:
    lib = _native.lib()
    m_p, k_p = qa.padded_shape
    n_p = qb.padded_shape[0]
    m, n = qa.original_shape[0], qb.original_shape[0]
    head = (qa.values.data_ptr(), qa.scale_factors.data_ptr(), _native.FOS_IF4, _native.FOS_SF_ROWMAJOR,
            qb.values.data_ptr(), qb.scale_factors.data_ptr(), _native.FOS_IF4, _native.FOS_SF_ROWMAJOR,
            alpha.data_ptr(), out.data_ptr(), _native.FOS_BF16, m_p, n_p, k_p, m, n, out.stride(0))
    stream = _native.stream_ptr(out.device)
    if static:
        return lib.fos_gemm_if4_static(*head, 0, stream)
    return lib.fos_gemm_if4(*head, workspace.data_ptr(), workspace.numel(), 0, stream)


def test_static_workspace_entry_matches_the_workspace_entry_twice():
    lib = _native.lib()
    for seed, (m, n, k) in enumerate([(384, 640, 448), (1024, 512, 2048)]):
        qa, qb = _operands(100 + seed, m, n, k)
        alpha = torch.empty(1, dtype=torch.float32, device=DEV)
        assert lib.fos_gemm_alpha(qa.amax.data_ptr(), _native.FOS_IF4, qa.scale_rule.cuda_id, qb.amax.data_ptr(),
                                  _native.FOS_IF4, qb.scale_rule.cuda_id, alpha.data_ptr(),
                                  _native.stream_ptr(alpha.device)) == 0
        nbytes = int(lib.fos_gemm_if4_workspace_bytes(*qa.padded_shape[:1], qb.padded_shape[0], qa.padded_shape[1]))
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert _call(False, qa, qb, want, alpha, workspace) == 0
        if seed == 0:
            assert _call(True, qa, qb, got, alpha) == 0        # the first call on a device does the one-time set-up
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        assert _call(True, qa, qb, got, alpha) == 0
        torch.cuda.synchronize()
        # nothing was allocated, by the driver or by torch's caching allocator
        assert torch.cuda.mem_get_info()[0] == free_before
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before
        assert torch.isfinite(want.float()).all()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"case {seed}"


def test_static_workspace_entry_refuses_what_does_not_fit():
    # (m_p + n_p) * k_p * 2 bytes = 64 MiB > 32 MiB; the check comes before any pointer is used
    qa, qb = _operands(7, 128, 128, 64)
    alpha = torch.ones(1, dtype=torch.float32, device=DEV)
    out = torch.empty(128, 128, dtype=torch.bfloat16, device=DEV)
    lib = _native.lib()
    rc = lib.fos_gemm_if4_static(
        qa.values.data_ptr(), qa.scale_factors.data_ptr(), _native.FOS_IF4, _native.FOS_SF_ROWMAJOR,
        qb.values.data_ptr(), qb.scale_factors.data_ptr(), _native.FOS_IF4, _native.FOS_SF_ROWMAJOR,
        alpha.data_ptr(), out.data_ptr(), _native.FOS_BF16, 4096, 4096, 4096, 128, 128, 128, 0,
        _native.stream_ptr(out.device))
    assert rc == FOS_ERR_TOO_LARGE
    assert b"maximum" in lib.fos_status_string(rc)
