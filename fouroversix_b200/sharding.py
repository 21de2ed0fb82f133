"""Tensor-parallel sharding of the FP4 linear layers across the GPUs of one node.

The reference has no distributed code of its own; it runs tensor-parallel only inside
vLLM (`--tensor-parallel-size`, scripts/ptq/__main__.py:281-287), where each rank
quantizes ITS shard of a weight with that shard's own amax
(src/fouroversix/integrations/vllm_quantization.py:100-124).  This module provides the
same decomposition natively, one process per GPU over torch.distributed (NCCL):

  column parallel   W[N, K] is split by rows; rank r holds W[r*N/g : (r+1)*N/g].
                    y_r = x @ W_r^T is a slice of the output; no communication.
  row parallel      W is split by columns; rank r holds W[:, r*K/g : (r+1)*K/g] and
                    receives the matching slice of the activations (the output of a
                    column-parallel layer). Every rank computes a full-size partial
                    product; the partials are summed with an all-reduce.

For row-parallel layers the all-reduce of a [tokens, N] bf16 tensor costs more than the
shard's GEMM at large token counts, so the token dimension is cut into chunks: the
all-reduce of chunk i runs on a communication stream while the GEMM of chunk i+1 runs
on the compute stream.

A row-parallel layer that feeds a column-parallel one (o_proj -> gate / up, down_proj -> the next
block's qkv) can hand its output over as ROW SLABS instead of a full tensor (`scatter_output=True` /
`scattered_input=True`): the partial products are reduce-scattered (every rank ends with tokens / g
rows, half the link traffic of an all-reduce), the ranks agree on the slabs' common amax (4 bytes),
each quantizes its own slab with it - the bytes of those rows of the unsharded quantization - and
the PACKED slabs (0.5625 bytes per value instead of 2) are all-gathered. Nothing is quantized g
times over, and whatever works row by row (a norm, a residual) runs on the slab.

Two ways to obtain shards:
  * quantize each shard by itself (`quantize(w_shard)`), the reference's behaviour; or
  * slice an already quantized tensor (`slice_rows`, `slice_cols`): bit-identical to the
    unsharded tensor, amax and therefore alpha stay global.  Row slices and K slices of
    the 128x4-tiled scale array are plain views / one gather because tiles are stored
    row-group major.
"""

from __future__ import annotations

import contextlib
from collections.abc import Callable

import torch
import torch.distributed as dist
import torch.nn as nn

from fouroversix_b200 import _native
from fouroversix_b200.matmul import quantized_matmul
from fouroversix_b200.quantize import QuantizationConfig, QuantizedTensor, quantize
from fouroversix_b200.utils import DataType, RoundStyle

from .model.config import ModuleQuantizationConfig


def shard_bounds(size: int, rank: int, world: int, multiple: int) -> tuple[int, int]:
    """[lo, hi) of rank's equal share of `size`; the share must be a multiple of `multiple`."""
    if size % world:
        raise ValueError(f"cannot split {size} evenly over {world} ranks")
    part = size // world
    if part % multiple:
        raise ValueError(f"a shard of {part} is not a multiple of {multiple}")
    return rank * part, (rank + 1) * part


def slice_rows(q: QuantizedTensor, lo: int, hi: int) -> QuantizedTensor:
    """Rows [lo, hi) of a quantized tensor (multiples of 128) without requantizing."""
    if lo % 128 or hi % 128 or not 0 <= lo < hi <= q.padded_shape[0]:
        raise ValueError("row slices must be multiples of 128 inside the padded shape")
    cols_p = q.padded_shape[1]
    per_row_scales = cols_p // q.dtype.block_size
    sf = q.scale_factors.reshape(-1)
    # tiled: 128-row groups are contiguous runs of tiles of 512 bytes (four blocks wide); row-major: rows are
    sf = sf[lo * per_row_scales: hi * per_row_scales]
    rows = min(hi, q.original_shape[0]) - lo
    return QuantizedTensor(q.values[lo:hi], sf, q.amax, q.dtype, (rows, q.original_shape[1]), q.scale_rule,
                           q.round_style, (hi - lo, cols_p),
                           scale_factors_are_in_blackwell_layout=q.scale_factors_are_in_blackwell_layout)


def slice_cols(q: QuantizedTensor, lo: int, hi: int) -> QuantizedTensor:
    """Columns [lo, hi) of a quantized tensor (multiples of four blocks: 64 values, 128 for MXFP4)
    without requantizing."""
    rows_p, cols_p = q.padded_shape
    block = q.dtype.block_size
    unit = 4 * block                                      # columns covered by one 512-byte scale tile
    if lo % unit or hi % unit or not 0 <= lo < hi <= cols_p:
        raise ValueError(f"column slices must be multiples of {unit} inside the padded shape")
    values = q.values[:, lo // 2: hi // 2].contiguous()
    if q.scale_factors_are_in_blackwell_layout:
        tiles = q.scale_factors.reshape(rows_p // 128, cols_p // unit, 512)
        sf = tiles[:, lo // unit: hi // unit].contiguous().reshape(-1)
    else:
        sf = q.scale_factors.reshape(rows_p, cols_p // block)[:, lo // block: hi // block].contiguous().reshape(-1)
    cols = min(hi, q.original_shape[1]) - lo
    return QuantizedTensor(values, sf, q.amax, q.dtype, (q.original_shape[0], cols), q.scale_rule, q.round_style,
                           (rows_p, hi - lo),
                           scale_factors_are_in_blackwell_layout=q.scale_factors_are_in_blackwell_layout)


MatmulFn = Callable[..., torch.Tensor]


class TensorParallelLinear(nn.Module):
    """One rank's part of a column- or row-parallel FP4 linear layer (inference).

    `weight` is this rank's shard, either high precision (quantized here with the
    shard's own amax, like the reference under vLLM) or already a `QuantizedTensor`.
    `matmul_fn(x, w, input_config=..., out_dtype=...)` defaults to the FP4 GEMM; tests of
    the host logic substitute a CPU stand-in. `chunks` and `comm_sms` shape the overlap of a
    row-parallel layer: the tokens are cut into `chunks` pieces, and while pieces are in flight the
    GEMM leaves `comm_sms` SMs idle (a per-call argument of the GEMM), because a persistent grid on
    every SM would keep the collective's kernel waiting until the GEMM has finished. 32 is what NCCL's all-reduce launches on a
    pair of B200s; with fewer free SMs part of its grid still waits for the GEMM.
    """

    PEER_SCATTER_MAX_WORLD = 8      # group sizes up to which the peer-memory reduce-scatter is the default (measured on 2, 4 and 8)

    def __init__(self, weight: torch.Tensor | QuantizedTensor, config: ModuleQuantizationConfig, mode: str, *,
                 group: dist.ProcessGroup | None = None, bias: torch.Tensor | None = None, chunks: int = 4,
                 comm_sms: int = 32, fused: bool | None = None, peer_mode: str = "scatter",
                 scatter_output: bool = False, scattered_input: bool = False, peer_scatter: bool | None = None,
                 peer_gather: bool | None = None, matmul_fn: MatmulFn | None = None,
                 quantize_fn: Callable | None = None, amax_fn: Callable | None = None) -> None:
        super().__init__()
        if mode not in ("column", "row"):
            raise ValueError("mode must be 'column' or 'row'")
        self.mode, self.config, self.group, self.chunks = mode, config, group, max(1, chunks)
        self.comm_sms = max(0, comm_sms)
        # row-parallel exchange through peer memory (scatter from the GEMM's epilogue, then reduce + gather):
        # None = use it when the layer's shape favours it (below) and it can be set up, True = require it,
        # False = NCCL all-reduce beside the GEMM
        self.fused = fused
        # "scatter": the GEMM's epilogue stores its tiles into the owners' staging buffers while it runs,
        # then the owners reduce and store to every rank (fos_gemm_nvfp4_scatter + fos_reduce_gather);
        # "pull": plain GEMM into this rank's symmetric buffer, then ONE kernel that loads every rank's rows
        # of this rank's slab, adds them and stores the sums back to every rank (fos_allreduce_peer).
        # Either way every link direction carries (world - 1) / world of the output twice; only the scatter
        # hides half of that behind the GEMM, and only when the GEMM is long enough: on two B200s, 32768
        # tokens, down_proj (K 14336 per rank) 3.0-3.1 ms with NCCL, 2.7 scatter, 3.0-3.1 pull; o_proj
        # (K 4096 per rank) 1.50 NCCL, 1.59 scatter (its peer stores hold the short GEMM back), 1.48 pull.
        # With fused=None the scatter is taken when the GEMM is at least twice as long as its scatter.
        if peer_mode not in ("pull", "scatter"):
            raise ValueError("peer_mode must be 'pull' or 'scatter'")
        self.peer_mode = peer_mode
        # Row slabs between a row-parallel layer and the column-parallel layer after it (module docstring).
        # Rank r's slab of a [tokens, n] tensor cut into `chunks` pieces is [chunks][tokens / (chunks * g)][n]:
        # of every chunk of tokens / chunks rows, the r-th part (`scatter_rows` builds it from a full tensor).
        if scatter_output and mode != "row":
            raise ValueError("scatter_output belongs to a row-parallel layer")
        if scattered_input and mode != "column":
            raise ValueError("scattered_input belongs to a column-parallel layer")
        self.scatter_output, self.scattered_input = scatter_output, scattered_input
        # scatter_output layers: the reduce-scatter over peer memory (fos_reduce_scatter_peer: every rank loads its
        # slab's rows from all ranks' partial products and adds them) instead of NCCL's. None = when every rank can
        # set the symmetric buffers up and the group is no larger than PEER_SCATTER_MAX_WORLD; True = require it.
        self.peer_scatter = peer_scatter
        # scattered_input layers: the all-gather of the packed slabs over peer memory (fos_allgather_peer: every rank
        # copies all ranks' pieces out of their symmetric buffers) instead of NCCL's. Only when asked for (True): on
        # four B200s it measured slower than NCCL's all-gather (qkv_proj 0.68 against 0.60 ms, gate_proj 1.17 against
        # 1.10 ms: the extra copy into the symmetric buffers, a barrier, and pull kernels that share the SMs the
        # capped GEMM leaves), on two the same.
        self.peer_gather = peer_gather
        self._gather_peer: dict | None = None
        self._peer: dict | None = None
        self._matmul = matmul_fn or quantized_matmul
        self._quantize = quantize_fn or quantize
        self._amax = amax_fn
        self.weight = weight if isinstance(weight, QuantizedTensor) else self._quantize(weight, config.get_weight_config())
        self.bias = bias
        self._comm_stream: torch.cuda.Stream | None = None
        self._sms: int | None = None               # SM count of the device (looked up once)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def _sm_count(self, dev: torch.device) -> int:
        if self._sms is None:
            self._sms = torch.cuda.get_device_properties(dev).multi_processor_count
        return self._sms

    def _alpha_for(self, xq: QuantizedTensor) -> torch.Tensor | None:
        """alpha of `xq @ weight.T` (fos_gemm_alpha_ex), once per forward for all its chunks - or None when the row
        ranges of this activation do not go through the native calls of `_gemm_rows`."""
        w = self.weight
        if not (self._matmul is quantized_matmul and xq.values.is_cuda and xq.dtype == w.dtype == DataType.nvfp4
                and xq.scale_factors_are_in_blackwell_layout and w.scale_factors_are_in_blackwell_layout
                and w.padded_shape[1] == xq.padded_shape[1] and xq.values.is_contiguous()
                and xq.scale_factors.is_contiguous()):
            return None
        dev = xq.values.device
        alpha = torch.empty(1, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _native.check(_native.lib().fos_gemm_alpha_ex(
                xq.amax.data_ptr(), _native.FOS_NVFP4, xq.scale_rule.cuda_id, int(xq.round_style == RoundStyle.stochastic_unbiased),
                w.amax.data_ptr(), _native.FOS_NVFP4, w.scale_rule.cuda_id, int(w.round_style == RoundStyle.stochastic_unbiased),
                alpha.data_ptr(), _native.stream_ptr(dev)), "fos_gemm_alpha")
        return alpha

    def _gemm_rows(self, xq: QuantizedTensor, lo: int, hi: int, act_cfg: QuantizationConfig, out: torch.Tensor,
                   max_ctas: int = 0, alpha: torch.Tensor | None = None) -> torch.Tensor:
        """out = xq[lo:hi] @ weight.T for a row range on 128-row boundaries of a packed activation. With an `alpha`
        from `_alpha_for` this is the native GEMM call itself (fos_gemm_nvfp4_ex) on offsets into the packed
        buffers - the layers of a sharded stack are called thousands of times a second, and the front end's checks
        and the row-slice objects cost more host time than the call; anything else goes through `_gemm` on a
        `slice_rows` view."""
        w = self.weight
        rows = hi - lo
        if (alpha is None or lo % 128 or rows % 128 or out.stride(1) != 1 or out.shape != (rows, w.original_shape[0])
                or out.dtype != DataType(self.config.output_dtype).torch_dtype):
            return self._gemm(slice_rows(xq, lo, hi), act_cfg, out=out, max_ctas=max_ctas)
        dev = out.device
        k_p = xq.padded_shape[1]
        lib, stream = _native.lib(), _native.stream_ptr(dev)

        def launch() -> None:
            _native.check(lib.fos_gemm_nvfp4_ex(
                xq.values.data_ptr() + lo * (k_p // 2), xq.scale_factors.data_ptr() + lo * (k_p // 16),
                w.values.data_ptr(), w.scale_factors.data_ptr(), alpha.data_ptr(), out.data_ptr(),
                _native.elem_code(out.dtype), rows, w.padded_shape[0], k_p, rows, w.original_shape[0], out.stride(0),
                _native.gemm_opts(0, max_ctas), 0, stream), "fos_gemm_nvfp4")

        if dev.index is None or dev.index == torch.cuda.current_device():
            launch()
        else:
            with torch.cuda.device(dev):
                launch()
        return out

    def _gemm(self, x: torch.Tensor | QuantizedTensor, act_cfg: QuantizationConfig,
              out: torch.Tensor | None = None, max_ctas: int = 0) -> torch.Tensor:
        extra = {} if out is None else {"out": out}
        if max_ctas:
            extra["max_ctas"] = max_ctas          # per call: nothing process-wide is touched
        return self._matmul(x, self.weight, input_config=act_cfg, out_dtype=self.config.output_dtype, **extra)

    def forward(self, x: torch.Tensor | QuantizedTensor) -> torch.Tensor:
        act_cfg = self.config.get_activation_config()
        if isinstance(x, QuantizedTensor):
            # an activation that is already quantized (and, for scattered_input layers, already gathered):
            # layers that read the same activation (gate_proj / up_proj, or q / k / v kept apart) share one
            # quantization or one gather (`quantize_input`)
            if self.mode != "column" and self.world_size > 1:
                raise ValueError("a row-parallel layer quantizes its own K shard")
            out = self._gemm(x, act_cfg)
            return out if self.bias is None else out + self.bias
        lead = x.shape[:-1]
        x2d = x.reshape(-1, x.shape[-1])
        if self.world_size == 1:
            out = self._gemm(x2d, act_cfg)
        elif self.mode == "column":
            out = self._column_from_slab(x2d, act_cfg) if self.scattered_input else self._gemm(x2d, act_cfg)
        elif self.scatter_output:
            out = self._row_parallel_scattered(x2d, act_cfg)
        else:
            out = self._row_parallel(x2d, act_cfg)
        if self.bias is not None:
            if self.mode == "row" and self.scatter_output and self.world_size > 1:
                raise ValueError("a bias on a scattered output is the caller's to add (once, by the rows' owner)")
            out = out + self.bias
        if out.shape[0] != x2d.shape[0]:
            return out                    # slab hand-off: the rows are not the input's rows (2-D in, 2-D out)
        return out.reshape(*lead, out.shape[-1])

    def quantize_input(self, x: torch.Tensor) -> QuantizedTensor:
        """The quantized activation this column-parallel layer would build from `x` (the full activation, or this
        rank's row slab for a scattered_input layer): pass it to `forward` of every layer that reads the same
        activation."""
        act_cfg = self.config.get_activation_config()
        x2d = x.reshape(-1, x.shape[-1])
        if self.scattered_input and self.world_size > 1:
            return self._gather_quantized(x2d, act_cfg)
        return self._quantize(x2d, act_cfg)

    # ------------------------------------------------------------------ row slabs between two layers

    def _slab_chunks(self, tokens: int) -> int:
        """How many chunks a tensor of `tokens` rows is cut into for the slab hand-off: the largest number not
        above `chunks` for which every rank's part of a chunk is a whole number of 128-row blocks."""
        world, n_chunks = self.world_size, self.chunks
        while n_chunks > 1 and tokens % (128 * world * n_chunks):
            n_chunks -= 1
        if tokens % (128 * world * n_chunks):
            raise ValueError(f"the slab hand-off needs tokens ({tokens}) to be a multiple of 128 * world size")
        return n_chunks

    def _row_parallel_scattered(self, x2d: torch.Tensor, act_cfg: QuantizationConfig) -> torch.Tensor:
        """Row-parallel layer whose result stays scattered: per chunk of tokens the partial product, then a
        reduce-scatter of the chunk on the communication stream while the next chunk's GEMM runs. Returns this
        rank's slab [tokens / g, n] (layout: see __init__)."""
        world, tokens = self.world_size, x2d.shape[0]
        n_chunks = self._slab_chunks(tokens)
        step, piece = tokens // n_chunks, tokens // (n_chunks * world)
        n_out = self.weight.original_shape[0]
        dtype = DataType(self.config.output_dtype).torch_dtype
        xq = self._quantize(x2d, act_cfg)
        on_gpu = x2d.device.type == "cuda"
        # over peer memory when asked for, or when it can be had (a collective decision, taken once per shape)
        use_peer = False
        if (on_gpu and self.peer_scatter is not False and self._matmul is quantized_matmul and n_out % 8 == 0
                and dtype in (torch.bfloat16, torch.float16)
                and (self.peer_scatter or world <= self.PEER_SCATTER_MAX_WORLD)):
            use_peer = self._agree_on_peer_buffers(tokens, n_out, dtype, x2d.device, required=bool(self.peer_scatter))
            if not use_peer:
                self.peer_scatter = False
        elif self.peer_scatter:
            raise ValueError("TensorParallelLinear: this call does not fit the peer-memory reduce-scatter")
        partial = self._peer["out"] if use_peer else torch.empty(tokens, n_out, dtype=dtype, device=x2d.device)
        slab = torch.empty(n_chunks * piece, n_out, dtype=dtype, device=x2d.device)
        rank = dist.get_rank(self.group)
        works = []
        max_ctas = 0
        if on_gpu:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=x2d.device)
            compute = torch.cuda.current_stream(x2d.device)
            if self.comm_sms > 0 and n_chunks > 1:
                max_ctas = max(1, self._sm_count(x2d.device) - self.comm_sms)
        alpha = self._alpha_for(xq) if on_gpu else None
        for i in range(n_chunks):
            part = partial[i * step: (i + 1) * step]
            self._gemm_rows(xq, i * step, (i + 1) * step, act_cfg, part, max_ctas, alpha)
            mine = slab[i * piece: (i + 1) * piece]
            if on_gpu:
                done = torch.cuda.Event()
                done.record(compute)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(done)
                    if use_peer:
                        self._peer["h_out"].barrier(channel=0)       # every rank's GEMM of this chunk is complete
                        with torch.cuda.device(x2d.device):
                            _native.check(_native.lib().fos_reduce_scatter_peer(
                                self._peer["out_ptrs"], world, i * step + rank * piece, piece, n_out, n_out,
                                mine.data_ptr(), n_out, _native.elem_code(dtype), 0,
                                _native.stream_ptr(x2d.device)), "fos_reduce_scatter_peer")
                    else:
                        dist.reduce_scatter_tensor(mine, part, group=self.group)
            else:
                works.append(dist.reduce_scatter_tensor(mine, part, group=self.group, async_op=True))
        if on_gpu:
            # the compute stream now follows everything the communication stream did, so the buffers it used
            # can be reused in stream order (no record_stream: that would keep 512 MiB blocks from the
            # allocator's free list until the side stream's events are polled)
            if use_peer:
                with torch.cuda.stream(self._comm_stream):
                    self._peer["h_out"].barrier(channel=0)           # no rank overwrites its buffer while a peer reads it
            compute.wait_stream(self._comm_stream)
        for w in works:
            w.wait()
        return slab

    def _gather_quantized(self, slab: torch.Tensor, act_cfg: QuantizationConfig) -> QuantizedTensor:
        """The quantized full activation from every rank's row slab: the ranks take the maximum of their slabs'
        amax, each quantizes its slab with it (the bytes of those rows of the unsharded quantization: blocks of
        16 along a row depend on nothing else), and codes and scales are all-gathered chunk by chunk into the
        layout the GEMM reads."""
        xq, events = self._start_gather(slab, act_cfg)
        if events:
            compute = torch.cuda.current_stream(slab.device)
            for ev in events:
                compute.wait_event(ev)
        return xq

    def _start_gather(self, slab: torch.Tensor, act_cfg: QuantizationConfig):
        """Quantizes the slab and starts the all-gathers of its chunks on the communication stream. Returns the
        full QuantizedTensor (complete on a CPU group; on a GPU chunk i is complete once events[i] has fired)."""
        world = self.world_size
        if act_cfg.block_scale_2d or act_cfg.transpose or act_cfg.rht or DataType(act_cfg.dtype) != DataType.nvfp4:
            raise ValueError("the slab hand-off quantizes activations to NVFP4 with 1-D blocks, untransposed")
        rows, k = slab.shape
        tokens = rows * world
        n_chunks = self._slab_chunks(tokens)
        step, piece = tokens // n_chunks, rows // n_chunks
        if self._amax is not None:
            amax = self._amax(slab)
        else:
            from fouroversix_b200.quantize.backend import B200QuantizeBackend
            amax = B200QuantizeBackend.amax(slab)
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        if self._quantize is quantize:
            from fouroversix_b200.quantize.backend import B200QuantizeBackend
            q = B200QuantizeBackend.quantize(slab, act_cfg, amax=amax)
        else:
            q = self._quantize(slab, act_cfg, amax=amax)
        k_p = q.padded_shape[1]
        codes = torch.empty(tokens, k_p // 2, dtype=torch.uint8, device=slab.device)
        scales = torch.empty(tokens * k_p // 16, dtype=torch.uint8, device=slab.device)
        sf_local = q.scale_factors.view(torch.uint8).reshape(-1)
        per_row = k_p // 16                                  # scale bytes per row; 128-row groups are contiguous
        on_gpu = slab.device.type == "cuda"
        events = []
        # over peer memory when asked for, or when it can be had (a collective decision, taken once per shape)
        use_peer = False
        if on_gpu and self.peer_gather is True and self._quantize is quantize and q.values.shape[0] == rows:
            use_peer = self._agree_on_gather_buffers(rows, k_p, slab.device, required=bool(self.peer_gather))
            if not use_peer:
                self.peer_gather = False
        elif self.peer_gather:
            raise ValueError("TensorParallelLinear: this call does not fit the peer-memory all-gather")
        if on_gpu:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=slab.device)
            compute = torch.cuda.current_stream(slab.device)
            if use_peer:
                gp = self._gather_peer
                if gp["free"] is not None:
                    compute.wait_event(gp["free"])           # every rank has finished reading the previous slab
                gp["codes"].copy_(q.values)
                gp["scales"].copy_(sf_local)
            ready = torch.cuda.Event()
            ready.record(compute)
            self._comm_stream.wait_event(ready)
            if use_peer:
                with torch.cuda.stream(self._comm_stream):
                    gp["h_codes"].barrier(channel=0)         # every rank's packed slab is in its symmetric buffer
        # (one stream context around the whole loop: entering one per chunk costs host time the layer feels)
        with (torch.cuda.stream(self._comm_stream) if on_gpu else contextlib.nullcontext()):
            for i in range(n_chunks):
                src_codes = q.values[i * piece: (i + 1) * piece]
                src_sf = sf_local[i * piece * per_row: (i + 1) * piece * per_row]
                dst_codes = codes[i * step: (i + 1) * step]
                dst_sf = scales[i * step * per_row: (i + 1) * step * per_row]
                if on_gpu:
                    if use_peer:
                        with torch.cuda.device(slab.device):
                            lib, stream = _native.lib(), _native.stream_ptr(slab.device)
                            _native.check(lib.fos_allgather_peer(
                                gp["codes_ptrs"], world, i * piece * (k_p // 2), piece * (k_p // 2),
                                dst_codes.data_ptr(), 0, stream), "fos_allgather_peer")
                            _native.check(lib.fos_allgather_peer(
                                gp["scales_ptrs"], world, i * piece * per_row, piece * per_row,
                                dst_sf.data_ptr(), 0, stream), "fos_allgather_peer")
                    else:
                        dist.all_gather_into_tensor(dst_codes, src_codes, group=self.group)
                        dist.all_gather_into_tensor(dst_sf, src_sf, group=self.group)
                    ev = torch.cuda.Event()
                    ev.record(self._comm_stream)
                    events.append(ev)
                else:
                    dist.all_gather_into_tensor(dst_codes, src_codes.contiguous(), group=self.group)
                    dist.all_gather_into_tensor(dst_sf, src_sf.contiguous(), group=self.group)
        if use_peer:
            with torch.cuda.stream(self._comm_stream):
                gp["h_codes"].barrier(channel=0)             # nobody overwrites its slab while a peer still reads it
                gp["free"] = torch.cuda.Event()
                gp["free"].record(self._comm_stream)
        # (callers wait for the last event on the compute stream before they return, which orders every later
        # use of these buffers after the gathers)
        xq = QuantizedTensor(codes, scales.view(q.scale_factors.dtype), amax, q.dtype, (tokens, k), q.scale_rule,
                             q.round_style, (tokens, k_p),
                             scale_factors_are_in_blackwell_layout=q.scale_factors_are_in_blackwell_layout)
        return xq, events

    def _column_from_slab(self, slab: torch.Tensor, act_cfg: QuantizationConfig) -> torch.Tensor:
        """Column-parallel layer fed by row slabs: the GEMM of chunk i runs as soon as its packed rows have been
        gathered, while the gathers of the later chunks are still on the links."""
        xq, events = self._start_gather(slab, act_cfg)
        if len(events) <= 1:
            if events:
                torch.cuda.current_stream(slab.device).wait_event(events[0])
            return self._gemm(xq, act_cfg)
        tokens = xq.original_shape[0]
        step = tokens // len(events)
        n_out = self.weight.original_shape[0]
        out = torch.empty(tokens, n_out, dtype=DataType(self.config.output_dtype).torch_dtype, device=slab.device)
        compute = torch.cuda.current_stream(slab.device)
        max_ctas = 0
        if self.comm_sms > 0 and self._matmul is quantized_matmul:
            max_ctas = max(1, self._sm_count(slab.device) - self.comm_sms)
        alpha = self._alpha_for(xq)
        for i, ev in enumerate(events):
            compute.wait_event(ev)
            last = i + 1 == len(events)
            self._gemm_rows(xq, i * step, (i + 1) * step, act_cfg, out[i * step: (i + 1) * step], 0 if last else max_ctas, alpha)
        return out

    def _peer_buffers(self, tokens: int, n_out: int, dtype: torch.dtype, dev: torch.device) -> dict:
        """Staging [world][tokens / world][n_out] and output [tokens][n_out] of this rank in symmetric
        memory (every rank maps every rank's buffers), built once per shape."""
        key = (tokens, n_out, dtype)
        if self._peer is not None and self._peer["key"] == key:
            return self._peer
        import ctypes

        import torch.distributed._symmetric_memory as symm

        world = self.world_size
        group = self.group if self.group is not None else dist.group.WORLD
        def pointers(handle):
            return (ctypes.c_void_p * world)(*[int(ptr) for ptr in handle.buffer_ptrs])

        out = symm.empty((tokens, n_out), dtype=dtype, device=dev)
        h_out = symm.rendezvous(out, group)
        self._peer = {"key": key, "out": out, "h_out": h_out, "out_ptrs": pointers(h_out)}
        if self.peer_mode == "scatter" and not self.scatter_output:
            staging = symm.empty((world, tokens // world, n_out), dtype=dtype, device=dev)
            h_staging = symm.rendezvous(staging, group)
            self._peer.update(staging=staging, h_staging=h_staging, staging_ptrs=pointers(h_staging))
        return self._peer

    def _agree_on_gather_buffers(self, rows: int, k_p: int, dev: torch.device, *, required: bool) -> bool:
        """Symmetric buffers for this rank's packed slab (codes [rows, k_p / 2], scales rows * k_p / 16 bytes), set up
        once per shape; the ranks agree on whether ALL of them could (see _agree_on_peer_buffers)."""
        key = (rows, k_p)
        if self._gather_peer is not None and self._gather_peer["key"] == key:
            return True
        failure: Exception | None = None
        buf: dict | None = None
        try:
            import ctypes

            import torch.distributed._symmetric_memory as symm

            world = self.world_size
            group = self.group if self.group is not None else dist.group.WORLD

            def pointers(handle):
                return (ctypes.c_void_p * world)(*[int(ptr) for ptr in handle.buffer_ptrs])

            codes = symm.empty((rows, k_p // 2), dtype=torch.uint8, device=dev)
            h_codes = symm.rendezvous(codes, group)
            scales = symm.empty((rows * k_p // 16,), dtype=torch.uint8, device=dev)
            h_scales = symm.rendezvous(scales, group)
            buf = {"key": key, "codes": codes, "h_codes": h_codes, "codes_ptrs": pointers(h_codes),
                   "scales": scales, "h_scales": h_scales, "scales_ptrs": pointers(h_scales), "free": None}
        except Exception as exc:                           # symmetric memory is not available here
            failure = exc
        ok = torch.tensor([0 if failure else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self._gather_peer = None
            if required:
                raise RuntimeError("TensorParallelLinear: the peer-memory all-gather could not be set up on every "
                                   "rank") from failure
            return False
        self._gather_peer = buf
        return True

    def _agree_on_peer_buffers(self, tokens: int, n_out: int, dtype: torch.dtype, dev: torch.device, *,
                               required: bool) -> bool:
        """Sets the symmetric buffers up (once per shape) and lets the ranks agree on whether ALL of them could:
        one that falls back to NCCL while the others wait at a symmetric-memory barrier would hang the group."""
        key = (tokens, n_out, dtype)
        if self._peer is not None and self._peer["key"] == key:
            return True
        failure: Exception | None = None
        try:
            self._peer_buffers(tokens, n_out, dtype, dev)
        except Exception as exc:                           # symmetric memory is not available here
            failure = exc
        ok = torch.tensor([0 if failure else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self._peer = None
            if required:
                raise RuntimeError("TensorParallelLinear: the peer-memory exchange could not be set up on every "
                                   "rank") from failure
            return False
        return True

    def _row_parallel_fused(self, x2d: torch.Tensor, act_cfg: QuantizationConfig) -> torch.Tensor | None:
        """The exchange over peer memory, in one of two forms (`peer_mode`). "pull": the GEMM stores this rank's
        partial product into its symmetric buffer, a barrier, one kernel loads the rows of this rank's slab from
        every rank, adds them and stores the sums into every rank's buffer (fos_allreduce_peer), a barrier.
        "scatter": the GEMM's epilogue scatters this rank's partial tiles into the
        owners' staging buffers while the GEMM runs (fos_gemm_nvfp4_scatter), a barrier, every rank reduces
        its slab and stores it into every rank's output (fos_reduce_gather), a barrier. Returns None when the
        request does not fit (the caller then takes the NCCL path). The result lives in a buffer that the
        next call of this layer overwrites."""
        from fouroversix_b200.matmul.backend import B200MatmulBackend

        world, tokens = self.world_size, x2d.shape[0]
        n_out = self.weight.original_shape[0]
        out_dtype = DataType(self.config.output_dtype)
        if (self._matmul is not quantized_matmul or x2d.device.type != "cuda" or not 2 <= world <= 8
                or tokens % (128 * world) or n_out % 8 or out_dtype not in (DataType.bfloat16, DataType.float16)
                or self.weight.dtype != DataType.nvfp4 or act_cfg.dtype != DataType.nvfp4
                or not self.weight.scale_factors_are_in_blackwell_layout):
            return None
        if self.fused is None:
            # GEMM time / scatter time ~ K_local * 1.5e-4 * world / (world - 1)  (4 PFLOP/s against 600 GB/s)
            k_local = self.weight.original_shape[1]
            if k_local * 1.5e-4 * world / (world - 1) < 2.0:
                return None
        # Every rank must take the same path: one that falls back to NCCL while the others wait at a
        # symmetric-memory barrier would hang the group. So the ranks agree (once per shape) on whether
        # ALL of them could set the buffers up.
        if not self._agree_on_peer_buffers(tokens, n_out, out_dtype.torch_dtype, x2d.device, required=bool(self.fused)):
            self.fused = False
            return None
        buf = self._peer
        rank = dist.get_rank(self.group)
        xq = self._quantize(x2d, act_cfg)
        if self.peer_mode == "pull":
            B200MatmulBackend.quantized_matmul(xq, self.weight, out_dtype=out_dtype, out=buf["out"])
            buf["h_out"].barrier(channel=0)                # every rank's partial product is complete
            with torch.cuda.device(x2d.device):
                _native.check(_native.lib().fos_allreduce_peer(
                    buf["out_ptrs"], world, rank, tokens, n_out, n_out, _native.elem_code(out_dtype.torch_dtype),
                    _native.stream_ptr(x2d.device)), "fos_allreduce_peer")
            buf["h_out"].barrier(channel=0)                # every slab of my buffer holds the sums
            return buf["out"]
        B200MatmulBackend.quantized_matmul_scatter(xq, self.weight, out_dtype=out_dtype, d_peers=buf["staging_ptrs"],
                                                   world=world, rank=rank)
        buf["h_staging"].barrier(channel=0)                # every rank's plane of my slab has arrived
        with torch.cuda.device(x2d.device):
            _native.check(_native.lib().fos_reduce_gather(
                buf["staging"].data_ptr(), buf["out_ptrs"], world, rank, tokens // world, n_out, n_out, n_out,
                _native.elem_code(out_dtype.torch_dtype), _native.stream_ptr(x2d.device)), "fos_reduce_gather")
        buf["h_out"].barrier(channel=0)                    # every slab of my output is in
        return buf["out"]

    def _row_parallel(self, x2d: torch.Tensor, act_cfg: QuantizationConfig) -> torch.Tensor:
        """Partial product per chunk of tokens, each chunk's all-reduce overlapped with the
        next chunk's GEMM. The local activations are quantized once (one amax for all
        chunks) and sliced by rows."""
        if self.fused is not False:
            out = self._row_parallel_fused(x2d, act_cfg)
            if out is not None:
                return out
            if self.fused:
                raise ValueError("TensorParallelLinear: this call does not fit the peer-memory exchange "
                                 "(NVFP4 operands, bf16 / fp16 output, tokens a multiple of 128 * world size)")
        tokens = x2d.shape[0]
        n_chunks = self.chunks
        while n_chunks > 1 and (tokens % (128 * n_chunks) != 0):
            n_chunks -= 1
        xq = self._quantize(x2d, act_cfg)
        on_gpu = x2d.device.type == "cuda"
        if n_chunks == 1:
            out = self._gemm(xq, act_cfg)
            dist.all_reduce(out, group=self.group)
            return out
        step = tokens // n_chunks
        n_out = self.weight.original_shape[0]
        out = torch.empty(tokens, n_out, dtype=DataType(self.config.output_dtype).torch_dtype, device=x2d.device)
        works = []
        if on_gpu:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=x2d.device)
            compute = torch.cuda.current_stream(x2d.device)
        max_ctas = 0
        if on_gpu and self.comm_sms > 0 and self._matmul is quantized_matmul:
            max_ctas = max(1, self._sm_count(x2d.device) - self.comm_sms)
        alpha = self._alpha_for(xq) if on_gpu else None
        for i in range(n_chunks):
            part = out[i * step: (i + 1) * step]
            self._gemm_rows(xq, i * step, (i + 1) * step, act_cfg, part, max_ctas, alpha)
            if on_gpu:
                done = torch.cuda.Event()
                done.record(compute)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(done)
                    dist.all_reduce(part, group=self.group)
            else:
                works.append(dist.all_reduce(part, group=self.group, async_op=True))
        if on_gpu:
            compute.wait_stream(self._comm_stream)
        for w in works:
            w.wait()
        return out


def scatter_rows(x: torch.Tensor, rank: int, world: int, chunks: int = 1) -> torch.Tensor:
    """Rank `rank`'s row slab of a full [tokens, n] tensor in the layout of the slab hand-off: of every
    chunk of tokens / chunks rows the rank-th part, the parts stacked in chunk order."""
    tokens = x.shape[0]
    if tokens % (chunks * world):
        raise ValueError(f"{tokens} rows do not split into {chunks} chunks of {world} parts")
    piece = tokens // (chunks * world)
    return x.reshape(chunks, world, piece, *x.shape[1:])[:, rank].reshape(chunks * piece, *x.shape[1:])


def gather_rows(slabs: list[torch.Tensor], chunks: int = 1) -> torch.Tensor:
    """Inverse of `scatter_rows`: the full tensor from the slabs of all ranks (rank order)."""
    world = len(slabs)
    piece = slabs[0].shape[0] // chunks
    stacked = torch.stack([t.reshape(chunks, piece, *t.shape[1:]) for t in slabs], dim=1)   # [chunks, world, piece, ...]
    return stacked.reshape(chunks * world * piece, *slabs[0].shape[1:])


def shard_linear_weight(weight: torch.Tensor, mode: str, rank: int, world: int) -> torch.Tensor:
    """The slice of a full [N, K] weight that `rank` owns in a `mode`-parallel layer."""
    n, k = weight.shape
    if mode == "column":
        lo, hi = shard_bounds(n, rank, world, 128)
        return weight[lo:hi]
    lo, hi = shard_bounds(k, rank, world, 64)
    return weight[:, lo:hi]
