"""Host logic of the tensor-parallel layers, on CPU with world_size 2 over gloo.

The FP4 kernels need a GPU, so the layers are given CPU stand-ins for `quantize` and
`quantized_matmul` built from the oracle; what is under test is the sharding arithmetic
(which rows / columns / scale tiles a rank owns), the chunked row-parallel all-reduce and
its agreement with the unsharded computation.
"""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import fouroversix_b200 as fos
from fouroversix_b200.sharding import (TensorParallelLinear, shard_bounds, shard_linear_weight, slice_cols,
                                       slice_rows)
from oracle import fos_oracle


def cpu_quantize(x: torch.Tensor, config: fos.QuantizationConfig) -> fos.QuantizedTensor:
    ref = fos_oracle.quantize(x.contiguous(), dtype=config.dtype, scale_rule=config.scale_rule,
                              block_scale_2d=config.block_scale_2d, transpose=config.transpose)
    return fos.QuantizedTensor(ref.values, ref.scale_factors.view(torch.float8_e4m3fn), ref.amax, config.dtype,
                               ref.original_shape, config.scale_rule, config.round_style, ref.padded_shape,
                               scale_factors_are_in_blackwell_layout=ref.tiled)


def cpu_dequantize(q: fos.QuantizedTensor, dtype=torch.float32) -> torch.Tensor:
    return fos_oracle.dequantize_raw(q.values, q.scale_factors, q.amax, q.dtype, q.scale_rule, q.original_shape,
                                     dtype, tiled=q.scale_factors_are_in_blackwell_layout)


def cpu_matmul(x, w, *, input_config=None, out_dtype=fos.DataType.bfloat16, out=None, **_):
    if isinstance(x, torch.Tensor):
        x = cpu_quantize(x, input_config or fos.QuantizationConfig())
    res = (cpu_dequantize(x) @ cpu_dequantize(w).T).to(fos.DataType(out_dtype).torch_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def test_slices_equal_slices_of_the_dequantized_tensor():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(384, 256, generator=g).bfloat16()
    for cfg in (fos.QuantizationConfig(), fos.QuantizationConfig(dtype="if4")):
        q = cpu_quantize(x, cfg)
        full = cpu_dequantize(q)
        assert torch.equal(cpu_dequantize(slice_rows(q, 128, 384)), full[128:384])
        assert torch.equal(cpu_dequantize(slice_cols(q, 64, 192)), full[:, 64:192])
        both = slice_cols(slice_rows(q, 0, 256), 128, 256)
        assert torch.equal(cpu_dequantize(both), full[0:256, 128:256])
    with pytest.raises(ValueError):
        slice_rows(q, 64, 128)
    with pytest.raises(ValueError):
        slice_cols(q, 0, 96)
    assert shard_bounds(1024, 1, 4, 128) == (256, 512)
    with pytest.raises(ValueError):
        shard_bounds(1024, 0, 3, 128)
    with pytest.raises(ValueError):
        shard_bounds(256, 0, 4, 128)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        g = torch.Generator().manual_seed(1)
        tokens, hidden, inner = 512, 256, 512
        x = torch.randn(tokens, hidden, generator=g).bfloat16()
        w_up = (torch.randn(inner, hidden, generator=g) * 0.05).bfloat16()      # column parallel
        w_down = (torch.randn(hidden, inner, generator=g) * 0.05).bfloat16()    # row parallel
        cfg = fos.ModuleQuantizationConfig(output_dtype="float32")
        kw = dict(matmul_fn=cpu_matmul, quantize_fn=cpu_quantize)
        up = TensorParallelLinear(shard_linear_weight(w_up, "column", rank, world), cfg, "column", **kw)
        down = TensorParallelLinear(shard_linear_weight(w_down, "row", rank, world), cfg, "row", chunks=2, **kw)
        h = up(x)                                        # [tokens, inner / world], stays sharded
        assert h.shape == (tokens, inner // world)
        y = down(h.bfloat16())                           # all-reduced: identical on every rank

        # the same computation without torch.distributed: per-shard products summed in fp32
        want = torch.zeros(tokens, hidden)
        for r in range(world):
            h_r = cpu_matmul(x, cpu_quantize(shard_linear_weight(w_up, "column", r, world), cfg.get_weight_config()),
                             out_dtype=fos.DataType.float32).bfloat16()
            want += cpu_matmul(h_r, cpu_quantize(shard_linear_weight(w_down, "row", r, world).contiguous(),
                                                 cfg.get_weight_config()), out_dtype=fos.DataType.float32)
        err = ((y - want).abs().max() / want.abs().max()).item()
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        results[rank] = (err, same, tuple(y.shape))
    finally:
        dist.destroy_process_group()


def test_column_then_row_parallel_matches_unsharded_sum():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    for r in range(world):
        err, same, shape = results[r]
        assert shape == (512, 256)
        assert same, "ranks disagree after the all-reduce"
        assert err < 1e-5, err


def test_layer_rejects_unknown_exchange_and_column_slices_follow_the_block_size():
    w = torch.randn(128, 128).bfloat16()
    with pytest.raises(ValueError, match="peer_mode"):
        TensorParallelLinear(w, fos.ModuleQuantizationConfig(), "row", peer_mode="ring", quantize_fn=cpu_quantize)
    with pytest.raises(ValueError, match="mode"):
        TensorParallelLinear(w, fos.ModuleQuantizationConfig(), "diagonal", quantize_fn=cpu_quantize)
    # MXFP4: a 512-byte scale tile covers 128 columns, so column slices come in multiples of 128
    ref = fos_oracle.quantize(torch.randn(128, 256).bfloat16(), dtype="mxfp4", scale_rule="static_6")
    q = fos.QuantizedTensor(ref.values, ref.scale_factors.view(torch.float8_e8m0fnu), ref.amax, "mxfp4", ref.original_shape,
                            "static_6", "nearest", ref.padded_shape, scale_factors_are_in_blackwell_layout=True)
    right = slice_cols(q, 128, 256)
    assert right.padded_shape == (128, 128) and right.scale_factors.numel() == 128 * 128 // 32
    assert torch.equal(right.values, q.values[:, 64:])
    full = fos_oracle.dequantize_raw(q.values, q.scale_factors, q.amax, "mxfp4", "static_6", (128, 256), torch.float32, tiled=True)
    part = fos_oracle.dequantize_raw(right.values, right.scale_factors, right.amax, "mxfp4", "static_6", (128, 128), torch.float32,
                                     tiled=True)
    assert torch.equal(part, full[:, 128:])
    with pytest.raises(ValueError, match="multiples of 128"):
        slice_cols(q, 64, 128)
