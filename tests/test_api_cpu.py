"""CPU-only checks: the C-ABI library loads and exports what include/*.h declares, and the
host-side mirror of the reference API behaves like the reference's."""

from __future__ import annotations

import re
from pathlib import Path

import pytest
import torch
import torch.nn as nn

import fouroversix_b200 as fos
from fouroversix_b200 import _native
from fouroversix_b200.quantize import from_blocked, to_blocked

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "fouroversix_b200.h").read_text()
    declared = set(re.findall(r"\b(fos_[a-z0-9_]+)\s*\(", header))
    assert {"fos_quantize", "fos_dequantize", "fos_gemm_nvfp4", "fos_gemm_alpha"} <= declared
    lib = _native.lib()
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    # the Python binding table and the header agree
    assert declared == set(_native.SIGNATURES), declared ^ set(_native.SIGNATURES)
    assert lib.fos_version() >= 200
    assert lib.fos_status_string(0) == b"ok"
    assert b"invalid" in lib.fos_status_string(-1)


def test_argument_validation_needs_no_gpu():
    lib = _native.lib()
    # NULL pointers and bad enums are rejected before any CUDA call
    assert lib.fos_quantize(0, 0, 128, 64, 64, 0, 3, 0, 0, 1, 0, 0, 0, 0, 0, 0) == -1
    # a kernel variant that does not exist is rejected before anything else is looked at
    bad = _native.GemmOpts(192, 0)
    import ctypes
    assert lib.fos_gemm_nvfp4_ex(0, 0, 0, 0, 0, 0, 0, 128, 128, 64, 128, 128, 128, ctypes.byref(bad), 0, 0) == -1
    assert not hasattr(lib, "fos_set_option")      # the library has no process-wide settings
    # grouped entries: NULL buffers, too many groups
    assert lib.fos_quantize_grouped(0, 0, 128, 64, 64, 0, 3, 0, 0, 4, 0, 0, 0, 0, 0, 0) == -1
    assert lib.fos_gemm_nvfp4_grouped(0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 128, 128, 64, 128, 128, 0, 0, 0) == -1
    assert lib.fos_gemm_alpha_grouped(0, 0, 3, 0, 0, 0, 3, 0, 0, 0, 0) == -1
    # experts entries: NULL buffers; the workspace size is plain host arithmetic
    assert lib.fos_experts_route(0, 8, 16, 2, 4, 1024, 0, 0, 0, 0, 0, 0, 0, 0) == -1
    assert lib.fos_experts_gather_rows(0, 0, 64, 0, 0, 64, 128, 64, 0, 0, 0) == -1
    assert lib.fos_experts_glu(0, 0, 128, 0, 0, 0, 64, 128, 64, 1.702, 7.0, 0, 0) == -1
    assert lib.fos_experts_combine(0, 0, 64, 0, 0, 0, 0, 2, 0, 64, 16, 64, 0) == -1
    assert lib.fos_experts_forward(*([0] * 19), 1, 1, 1.702, 7.0, 0, 0, 0, 0, 0, 0) == -1
    need = lib.fos_experts_workspace_bytes(256, 4, 32, 2880, 2880)
    capacity = (256 * 4 + 127 * 32 + 127) // 128 * 128
    assert need % 256 == 0 and need >= capacity * (2 * 2880 * 2 + 2 * 2 * 2880 + 2 * 2880 + 2 * (2880 // 2 + 2880 // 16))
    assert lib.fos_experts_workspace_bytes(0, 4, 32, 2880, 2880) == -1
    # a linear layer as one call: NULL buffers; the workspace holds the packed activation of the padded shape
    assert lib.fos_linear_forward(0, 0, 16, 8192, 8192, 3, 0, 0, 0, 3, 8192, 0, 0, 8192, 0, 0, None, 0, 0) == -1
    need = lib.fos_linear_workspace_bytes(16, 8200)
    assert need % 256 == 0 and need >= 128 * 8256 // 2 + 128 * 8256 // 16 + 8
    assert lib.fos_linear_workspace_bytes(16, 0) == -1


def test_group_layout_is_computed_without_reading_the_counts_back():
    import torch

    from fouroversix_b200.matmul import GroupLayout

    layout = GroupLayout.from_counts(torch.tensor([5, 0, 300, 128]), 433)
    assert layout.group_start.tolist() == [0, 128, 128, 512, 640] and layout.group_start.dtype == torch.int32
    assert layout.group_rows.tolist() == [5, 0, 300, 128]
    assert layout.capacity == 1024 and layout.capacity >= 640        # worst case for 433 rows in 4 groups
    with pytest.raises(ValueError):
        GroupLayout.from_counts(torch.zeros(300, dtype=torch.int64), 0)


def test_enums_and_config_coercion():
    cfg = fos.QuantizationConfig(dtype="if4", scale_rule="mae", round_style="nearest", backend="cuda")
    assert cfg.dtype is fos.DataType.if4 and cfg.scale_rule is fos.ScaleRule.mae
    assert cfg.backend is fos.QuantizeBackend.cuda
    assert fos.QuantizationConfig().scale_rule is fos.ScaleRule.mse
    assert fos.ScaleRule.mse.cuda_id == 3 and fos.ScaleRule.static_6.cuda_id == 0
    assert fos.DataType.nvfp4.block_size == 16 and fos.DataType.mxfp4.block_size == 32
    assert fos.DataType.if4.supported_scale_rules == {fos.ScaleRule.mse, fos.ScaleRule.mae, fos.ScaleRule.abs_max}
    assert fos.DataType.nvfp4.scale_type.get_maximum_value(fos.ScaleRule.mse) == 256
    assert fos.DataType.nvfp4.scale_type.get_maximum_value(fos.ScaleRule.static_6) == 448


def test_quantize_rejects_what_it_cannot_do():
    x = torch.zeros(128, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="No backend found"):
        fos.quantize(x)                                   # CPU tensor: there is no CPU path
    with pytest.raises(ValueError, match="does not support"):
        fos.quantize(x, fos.QuantizationConfig(backend="pytorch"))
    with pytest.raises(ValueError):
        fos.quantize(x, fos.QuantizationConfig(dtype="if4", scale_rule="static_6"))
    with pytest.raises(ValueError):
        fos.quantize(x.reshape(2, 64, 64))


def test_scale_tile_layout_round_trip():
    a = torch.arange(256 * 8, dtype=torch.int32).reshape(256, 8)
    b = to_blocked(a)
    assert torch.equal(from_blocked(b, (256, 8)), a)
    # element (r, c) of tile t sits at t*512 + (r%32)*16 + (r//32)*4 + c
    r, c = 77, 6
    off = ((r // 128) * 2 + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    assert b[off] == a[r, c]


def test_quantized_tensor_pads_like_the_reference():
    values = torch.zeros(100, 40, dtype=torch.uint8)
    scales = torch.ones(100, 5, dtype=torch.float32).to(torch.float8_e4m3fn)
    q = fos.QuantizedTensor(values, scales, torch.ones(1), "nvfp4", (100, 80), "mse", "nearest")
    assert q.padded_shape == (128, 128)
    assert q.values.shape == (128, 64) and q.scale_factors.numel() == 128 * 8
    with pytest.raises(ValueError):
        fos.QuantizedTensor(values, torch.ones(7).to(torch.float8_e4m3fn), torch.ones(1), "nvfp4", (100, 80),
                            "mse", "nearest")


def test_quantize_model_swaps_linear_layers():
    model = nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 64))
    model.add_module("lm_head", nn.Linear(64, 10))
    fos.quantize_model(model, fos.ModelQuantizationConfig(module_config_overrides={"2": {"scale_rule": "static_6"}}))
    assert isinstance(model[0], fos.FourOverSixLinear) and isinstance(model[2], fos.FourOverSixLinear)
    assert not isinstance(model.lm_head, fos.FourOverSixLinear)
    assert model[2].config.weight_scale_rule is fos.ScaleRule.static_6
    assert model[0].config.weight_scale_rule is fos.ScaleRule.mse
    sd = model[0].state_dict()
    assert sd["quantized_weight_values"].shape == (128, 32)
    assert sd["quantized_weight_scale_factors"].shape == (128 * 64 // 16,)
    assert sd["quantized_weight_metadata"].shape == (6,)
    with pytest.raises(ValueError):
        fos.QuantizedModule.register(nn.Linear)


def test_module_config_inherits_defaults():
    c = fos.ModuleQuantizationConfig(dtype="nvfp4", scale_rule="static_6", weight_scale_2d=True)
    assert c.get_weight_config(transpose=True) == fos.QuantizationConfig(
        block_scale_2d=True, scale_rule="static_6", transpose=True)
    assert c.get_gradient_config().round_style is fos.RoundStyle.stochastic
    assert isinstance(fos.ModelQuantizationConfig().__hash__(), str)


def test_backward_refuses_settings_it_does_not_implement():
    """Settings the reference's backward pass acts on (src/fouroversix/model/modules/linear.py:213-229,
    258-268) and this layer does not are refused, not silently ignored."""
    import torch

    from fouroversix_b200.model.linear import FourOverSixLinearFunction

    x, w, dy = torch.zeros(16, 64), torch.zeros(32, 64), torch.zeros(16, 32)
    for kwargs in (dict(wgrad_nvint4=True), dict(disable_dgrad_quantization="quantize_grad_only"),
                   dict(quartet_ii_dtype="nvfp4")):
        class Ctx:
            saved_tensors = (x, w, None)
            config = fos.ModuleQuantizationConfig(**kwargs)
            needs_input_grad = (False, True, True, False)

        with pytest.raises(NotImplementedError):
            FourOverSixLinearFunction.backward(Ctx, dy)


def test_experts_routing_tables_on_the_host():
    """The tensor-operation form of the experts layer's routing (`FourOverSixExperts.route`) needs no GPU: every
    (token, slot) pair gets a row of its expert's range, rows ascend with the pair inside an expert."""
    import torch

    from fouroversix_b200.model import FourOverSixExperts

    layer = FourOverSixExperts.__new__(FourOverSixExperts)
    torch.nn.Module.__init__(layer)
    layer.num_experts = 6
    g = torch.Generator().manual_seed(4)
    scores = torch.rand(37, 6, generator=g)
    scores[:, 2] = -1                                             # an expert nobody is routed to
    indices = torch.topk(scores, 3, dim=-1).indices
    layout, rows, token, order = layer.route(indices)
    flat = indices.reshape(-1)
    counts = torch.bincount(flat, minlength=6)
    assert layout.group_rows.tolist() == counts.tolist() and counts[2] == 0
    assert layout.group_start.tolist() == [0, *((counts + 127) // 128 * 128).cumsum(0).tolist()]
    expert = flat[order]
    start = layout.group_start.long()[expert]
    assert ((rows >= start) & (rows < start + counts[expert])).all() and rows.unique().numel() == rows.numel()
    assert torch.equal(token, order // 3)
    for e in range(6):
        mine, pairs = rows[expert == e], order[expert == e]
        assert (mine[1:] > mine[:-1]).all() and (pairs[1:] > pairs[:-1]).all()
