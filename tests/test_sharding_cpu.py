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
from fouroversix_b200.sharding import (TensorParallelLinear, gather_rows, scatter_rows, shard_bounds,
                                       shard_linear_weight, slice_cols, slice_rows)
from oracle import fos_oracle


def cpu_quantize(x: torch.Tensor, config: fos.QuantizationConfig, amax: torch.Tensor | None = None) -> fos.QuantizedTensor:
    ref = fos_oracle.quantize(x.contiguous(), dtype=config.dtype, scale_rule=config.scale_rule,
                              block_scale_2d=config.block_scale_2d, transpose=config.transpose, amax=amax)
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
        tokens, hidden, inner = 1024, 256, 512
        x = torch.randn(tokens, hidden, generator=g).bfloat16()
        w_up = (torch.randn(inner, hidden, generator=g) * 0.05).bfloat16()      # column parallel
        w_down = (torch.randn(hidden, inner, generator=g) * 0.05).bfloat16()    # row parallel
        w_next = (torch.randn(inner, hidden, generator=g) * 0.05).bfloat16()    # column parallel, fed by row slabs
        cfg = fos.ModuleQuantizationConfig(output_dtype="float32")
        kw = dict(matmul_fn=cpu_matmul, quantize_fn=cpu_quantize, amax_fn=lambda t: t.abs().max().float().reshape(1))
        up = TensorParallelLinear(shard_linear_weight(w_up, "column", rank, world), cfg, "column", **kw)
        w_down_shard = shard_linear_weight(w_down, "row", rank, world)
        down = TensorParallelLinear(w_down_shard, cfg, "row", chunks=2, **kw)
        h = up(x)                                        # [tokens, inner / world], stays sharded
        assert h.shape == (tokens, inner // world)
        y = down(h.bfloat16())                           # all-reduced: identical on every rank

        # the oracle's answer without torch.distributed: per-shard fp32 products (each shard quantized by itself,
        # with its own amax and alpha), row-parallel partials summed in fp32
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

        # the slab hand-off: the same row-parallel layer leaves its result scattered by rows, the next
        # column-parallel layer quantizes its slab with the common amax and gathers the packed slabs
        chunks = 2
        down_s = TensorParallelLinear(w_down_shard, cfg, "row", chunks=chunks, scatter_output=True, **kw)
        nxt = TensorParallelLinear(shard_linear_weight(w_next, "column", rank, world), cfg, "column", chunks=chunks,
                                   scattered_input=True, **kw)
        slab = down_s(h.bfloat16())
        slab_err = ((slab - scatter_rows(want, rank, world, chunks)).abs().max() / want.abs().max()).item()
        slabs = [torch.empty_like(slab) for _ in range(world)]
        dist.all_gather(slabs, slab)
        full = gather_rows(slabs, chunks).bfloat16()     # what an all-reduce would have left on every rank
        xq = nxt._gather_quantized(slab.bfloat16(), cfg.get_activation_config())
        ref = fos_oracle.quantize(full)                  # the unsharded quantization of the full activation
        packed_equal = (torch.equal(xq.values, ref.values) and torch.equal(xq.amax, ref.amax)
                        and torch.equal(xq.scale_factors.view(torch.uint8).flatten(), ref.scale_factors))
        z = nxt(slab.bfloat16())
        z_want = cpu_matmul(full, cpu_quantize(shard_linear_weight(w_next, "column", rank, world), cfg.get_weight_config()),
                            out_dtype=fos.DataType.float32)
        results[rank] = (err, same, tuple(y.shape), slab_err, packed_equal, torch.equal(z, z_want), tuple(slab.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_then_row_parallel_matches_unsharded_sum(world):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.terminate()
    assert not stuck, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs)
    for r in range(world):
        err, same, shape, slab_err, packed_equal, z_equal, slab_shape = results[r]
        assert shape == (1024, 256)
        assert same, "ranks disagree after the all-reduce"
        assert err < 1e-5, err                   # fp32 partials, fp32 sum: only the order of the additions differs
        assert slab_shape == (1024 // world, 256)
        assert slab_err < 1e-5, slab_err
        assert packed_equal, "slabs quantized with the common amax must carry the bytes of the unsharded quantization"
        assert z_equal


def test_scatter_and_gather_rows_are_inverse():
    x = torch.arange(48 * 3, dtype=torch.float32).reshape(48, 3)
    for world, chunks in ((2, 1), (4, 3), (3, 2)):
        slabs = [scatter_rows(x, r, world, chunks) for r in range(world)]
        assert slabs[0].shape == (48 // world, 3)
        assert torch.equal(gather_rows(slabs, chunks), x)
    # rank 1 of 2 with 2 chunks of 24 rows owns rows 12..23 and 36..47
    assert torch.equal(scatter_rows(x, 1, 2, 2)[:, 0] / 3, torch.cat([torch.arange(12, 24), torch.arange(36, 48)]).float())
    with pytest.raises(ValueError):
        scatter_rows(x, 0, 5, 1)


def test_layer_rejects_unknown_exchange_and_column_slices_follow_the_block_size():
    w = torch.randn(128, 128).bfloat16()
    with pytest.raises(ValueError, match="peer_mode"):
        TensorParallelLinear(w, fos.ModuleQuantizationConfig(), "row", peer_mode="ring", quantize_fn=cpu_quantize)
    with pytest.raises(ValueError, match="mode"):
        TensorParallelLinear(w, fos.ModuleQuantizationConfig(), "diagonal", quantize_fn=cpu_quantize)
    with pytest.raises(ValueError, match="scatter_output"):
        TensorParallelLinear(w, fos.ModuleQuantizationConfig(), "column", scatter_output=True, quantize_fn=cpu_quantize)
    with pytest.raises(ValueError, match="scattered_input"):
        TensorParallelLinear(w, fos.ModuleQuantizationConfig(), "row", scattered_input=True, quantize_fn=cpu_quantize)
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
