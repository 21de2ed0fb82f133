"""Scale-factor tile order used by Blackwell block-scaled MMA (host-side helpers).

A [rows, cols] matrix of per-block scales (rows a multiple of 128, cols a multiple of 4)
is cut into 128x4 tiles; each tile is stored as 512 contiguous bytes in which element
(r, c) sits at (r % 32) * 16 + (r // 32) * 4 + c.  Same layout as the reference's
`to_blocked` / `from_blocked` (src/fouroversix/quantize/utils.py:88-96,
src/fouroversix/quantize/dequantize_utils.py:4-12), computed here with one index gather.
The kernels write and read this order directly; these helpers serve padding, sharding
and tests.
"""

from __future__ import annotations

import functools

import torch


@functools.lru_cache(maxsize=64)
def _tiled_index(rows: int, cols: int) -> torch.Tensor:
    r = torch.arange(rows).unsqueeze(1)
    c = torch.arange(cols).unsqueeze(0)
    tile = (r // 128) * (cols // 4) + c // 4
    return (tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4).flatten()


def to_blocked(a: torch.Tensor) -> torch.Tensor:
    """Row-major [rows, cols] scales -> flat tensor in tile order."""
    rows, cols = a.shape
    if rows % 128 or cols % 4:
        raise ValueError("scale matrix must be a multiple of 128 rows and 4 columns")
    idx = _tiled_index(rows, cols).to(a.device)
    out = torch.empty(rows * cols, dtype=a.dtype, device=a.device)
    flat = a.reshape(-1)
    if a.dtype.itemsize == 1:
        out.view(torch.uint8)[idx] = flat.view(torch.uint8)
    else:
        out[idx] = flat
    return out


def from_blocked(a: torch.Tensor, orig_shape: tuple[int, int]) -> torch.Tensor:
    """Flat tile-ordered scales -> row-major [rows, cols]."""
    rows, cols = orig_shape
    idx = _tiled_index(rows, cols).to(a.device)
    flat = a.reshape(-1)
    if a.dtype.itemsize == 1:
        return flat.view(torch.uint8)[idx].view(a.dtype).reshape(rows, cols)
    return flat[idx].reshape(rows, cols)
