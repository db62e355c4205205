"""Float8 / MXFP8 numerics (PyTorch definition of the recipes) and converter behaviour."""

import dataclasses

import pytest
import torch

from torchtitan_b200.ops import quant


def test_fp8_quantize_round_trip_error_bounds():
    torch.manual_seed(0)
    x = torch.randn(64, 128) * 3
    for axis in (None, -1):
        q, s = quant.quantize_fp8(x, axis)
        assert q.dtype == torch.float8_e4m3fn
        back = q.float() * s
        # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normal values
        rel = ((back - x).abs() / x.abs().clamp_min(1e-3)).max()
        assert rel < 0.13, rel
    q, s = quant.quantize_fp8(x, -1)
    assert torch.equal(torch.log2(s), torch.log2(s).round())  # power-of-two rowwise scales


def test_mxfp8_scales_are_rceil_and_never_saturate():
    torch.manual_seed(0)
    x = torch.randn(8, 96) * torch.logspace(-3, 3, 8).view(8, 1)
    q, e = quant.quantize_mxfp8(x)
    assert q.shape == x.shape and e.shape == (8, 3) and e.dtype == torch.uint8
    amax = x.view(8, 3, 32).abs().amax(-1)
    expect = torch.ceil(torch.log2(amax / 448.0)) + 127
    assert torch.equal(e.float(), expect)
    assert q.float().abs().max() <= 448
    back = quant.dequantize_mxfp8(q, e)
    assert ((back - x).abs() / x.abs().clamp_min(1e-6)).median() < 0.05
    # column-major (axis 0) scaling for the weight-gradient operand
    q0, e0 = quant.quantize_mxfp8(x.t().contiguous(), axis=0)
    assert torch.equal(q0.t().float(), q.float()) and torch.equal(e0.t(), e)


@pytest.mark.parametrize("recipe", ["tensorwise", "rowwise", "rowwise_with_gw_hp", "mxfp8"])
def test_quant_linear_close_to_fp32(recipe):
    torch.manual_seed(1)
    x = torch.randn(4, 32, 64, requires_grad=True)
    w = (torch.randn(48, 64) * 0.1).requires_grad_()
    r = quant.QuantRecipe(kind="mxfp8") if recipe == "mxfp8" else quant.QuantRecipe(scaling=recipe, emulate=True)
    y = quant.quant_linear(x, w, None, r)
    y.square().sum().backward()
    gx, gw = x.grad.clone(), w.grad.clone()
    x.grad = w.grad = None
    yr = torch.nn.functional.linear(x, w)
    yr.square().sum().backward()

    def rel(a, b):
        return ((a - b).norm() / b.norm()).item()

    assert rel(y, yr) < 0.06 and rel(gx, x.grad) < 0.1 and rel(gw, w.grad) < 0.1, (rel(y, yr), rel(gx, x.grad), rel(gw, w.grad))


def test_float8_converter_selects_layers_and_trains():
    from torchtitan_b200.components.quantization.float8 import Float8LinearConverter
    from torchtitan_b200.models.llama3 import llama3_configs
    from torchtitan_b200.parallel import ParallelDims

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=1)
    conv = Float8LinearConverter.Config(emulate=True, filter_fqns=["output"]).build(parallel_dims=pd, model_compile_enabled=False)
    cfg = dataclasses.replace(llama3_configs["debugmodel"], n_layers=2)
    model = cfg.build()
    model.init_weights()
    conv.convert(model)
    assert model.output.quant is None and model.layers["0"].attention.wq.quant is not None
    keys_before = set(model.state_dict())
    x = torch.randint(0, cfg.vocab_size, (2, 32))
    model(x).float().logsumexp(-1).mean().backward()
    assert model.layers["0"].attention.wq.weight.grad is not None
    assert set(model.state_dict()) == keys_before
    with pytest.raises(ValueError):
        Float8LinearConverter.Config(emulate=False).build(parallel_dims=pd, model_compile_enabled=False)


def test_converters_of_different_quantization_types_are_rejected():
    from torchtitan_b200.components.quantization.float8 import Float8LinearConverter
    from torchtitan_b200.components.quantization.mx import MXFP8Converter
    from torchtitan_b200.parallel import ParallelDims
    from torchtitan_b200.protocols.model_converter import ModelConvertersContainer

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=1)
    cfg = ModelConvertersContainer.Config(converters=[Float8LinearConverter.Config(emulate=True), MXFP8Converter.Config(emulate=True)])
    with pytest.raises(ValueError, match="different quantization"):
        cfg.build(parallel_dims=pd, model_compile_enabled=False)


def test_mxfp8_converter_on_moe_experts():
    from torchtitan_b200.components.quantization.mx import MXFP8Converter
    from torchtitan_b200.models.qwen3 import qwen3_configs
    from torchtitan_b200.parallel import ParallelDims

    pd = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=1, pp=1, ep=1, etp=1, world_size=1)
    cfg = dataclasses.replace(qwen3_configs["debugmodel_moe"], n_layers=1)
    torch.manual_seed(0)
    model = cfg.build()
    model.init_weights()
    x = torch.randint(0, cfg.vocab_size, (2, 32))
    ref = model(x)
    MXFP8Converter.Config(fqns=["experts"], emulate=True).build(parallel_dims=pd, model_compile_enabled=False).convert(model)
    assert model.layers["0"].moe.experts.quant is not None
    out = model(x)
    out.float().logsumexp(-1).mean().backward()
    assert ((out - ref).norm() / ref.norm()) < 0.05
    assert model.layers["0"].moe.experts.w1.grad is not None
