"""Llama 4 / DeepSeek-V3 / gpt-oss: construction, one training step on CPU, Hugging Face name round trips."""

import dataclasses

import pytest
import torch


class _Tok:
    eos_id = 0


def _step(model, vocab, seq=64, bs=2, masks=True):
    torch.manual_seed(0)
    x = torch.randint(1, vocab, (bs, seq + 1))
    x[:, seq // 2] = 0  # one document boundary
    inp, lab = x[:, :-1], x[:, 1:]
    m = model.get_attention_masks(inp, _Tok()) if masks else None
    out = model(inp, m)
    assert out.shape == (bs, seq, vocab)
    loss = torch.nn.functional.cross_entropy(out.flatten(0, 1).float(), lab.flatten())
    loss.backward()
    missing = [n for n, p in model.named_parameters() if p.requires_grad and p.grad is None]
    return loss.item(), missing


def test_llama4_debugmodel_step_and_masks():
    from torchtitan_b200.models.llama4 import llama4_configs

    cfg = dataclasses.replace(llama4_configs["debugmodel"])          # a copy: the registry's object is shared by all tests
    cfg.layer = dataclasses.replace(cfg.layer, fixed_attn_block_size=16)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    model = cfg.build()
    model.init_weights()
    assert not model.layers["0"].attention.use_rope and model.layers["1"].attention.use_rope
    assert not model.layers["0"].moe_enabled and model.layers["1"].moe_enabled
    loss, missing = _step(model, cfg.vocab_size)
    assert loss == loss and not missing, missing


def test_llama4_fixed_block_mask_blocks_attention():
    """A RoPE layer must not see tokens of an earlier fixed block."""
    from torchtitan_b200.models.common.attention import AttentionMasks, InnerAttention

    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 32, 2, 16) for _ in range(3))
    inner = InnerAttention()
    a = inner(q, k, v, masks=AttentionMasks(block=8))
    k2, v2 = k.clone(), v.clone()
    k2[:, :8] += 1.0
    v2[:, :8] -= 1.0
    b = inner(q, k2, v2, masks=AttentionMasks(block=8))
    assert torch.allclose(a[:, 8:], b[:, 8:]) and not torch.allclose(a[:, :8], b[:, :8])


def test_llama4_hf_round_trip():
    from torchtitan_b200.models.llama4 import Llama4StateDictAdapter, llama4_configs

    cfg = dataclasses.replace(llama4_configs["debugmodel"], n_layers=2)
    model = cfg.build()
    model.init_weights()
    sd = {k: v for k, v in model.state_dict().items()}
    ad = Llama4StateDictAdapter(cfg, None)
    hf = ad.to_hf(sd)
    assert "language_model.model.layers.1.feed_forward.experts.gate_up_proj" in hf
    back = ad.from_hf(hf)
    for k, v in sd.items():
        if "expert_bias" in k:
            continue
        assert torch.equal(back[k], v), k


def test_deepseek_v3_debugmodel_step_and_adapter():
    from torchtitan_b200.models.deepseek_v3 import DeepSeekV3StateDictAdapter, deepseek_v3_configs

    cfg = dataclasses.replace(deepseek_v3_configs["debugmodel_flex_attn"], n_layers=3)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    model = cfg.build()
    model.init_weights(buffer_device=torch.device("cpu"))
    assert not model.layers["0"].moe_enabled and model.layers["1"].moe_enabled
    loss, missing = _step(model, cfg.vocab_size)
    assert loss == loss and not missing, missing
    sd = dict(model.state_dict())
    ad = DeepSeekV3StateDictAdapter(cfg, None)
    hf = ad.to_hf(sd)
    assert "model.layers.1.mlp.experts.7.down_proj.weight" in hf and "model.layers.1.mlp.gate.e_score_correction_bias" in hf
    back = ad.from_hf(hf)
    assert set(back) == set(sd)
    for k, v in sd.items():
        assert torch.equal(back[k], v), k


def test_deepseek_v3_mla_low_rank_query_and_yarn_scale():
    from torchtitan_b200.models.common import Linear, RMSNorm
    from torchtitan_b200.models.deepseek_v3 import Attention

    a = Attention.Config(n_heads=4, q_lora_rank=32, wq_a=Linear.Config(), wq_b=Linear.Config(), q_norm=RMSNorm.Config(),
                         kv_norm=RMSNorm.Config(), kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                         rope_factor=40.0, rope_max_seq_len=8192, rope_original_seq_len=4096, mscale=0.7).build(dim=128)
    import math

    m = 0.1 * 0.7 * math.log(40.0) + 1.0
    assert abs(a.softmax_scale - (48**-0.5) * m * m) < 1e-9
    assert hasattr(a, "wq_a") and not hasattr(a, "wq")


def test_block_fp8_dequantise():
    from torchtitan_b200.models.utils import dequantize_block_fp8

    w = torch.randn(200, 300)
    s = torch.rand(2, 3) + 0.5
    full = s.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300]
    q = (w / full).to(torch.float8_e4m3fn)
    assert torch.allclose(dequantize_block_fp8(q, s), q.float() * full)


def test_gpt_oss_debugmodel_step_sinks_window_and_adapter():
    from torchtitan_b200.models.gpt_oss import GptOssStateDictAdapter, gptoss_configs

    cfg = dataclasses.replace(gptoss_configs["debugmodel"], n_layers=2)
    cfg.rope = dataclasses.replace(cfg.rope, max_seq_len=64)
    cfg.layer = dataclasses.replace(cfg.layer, attention=dataclasses.replace(   # replace, not assign: the registry's object is shared
        cfg.layer.attention, n_heads=8, n_kv_heads=2, head_dim=32, sliding_window_size=8))
    cfg.rope = dataclasses.replace(cfg.rope, dim=32)
    model = cfg.build()
    model.init_weights(buffer_device=torch.device("cpu"))
    assert model.layers["0"].use_sliding_attention and not model.layers["1"].use_sliding_attention
    loss, missing = _step(model, cfg.vocab_size)
    assert loss == loss and not missing, missing
    assert model.layers["0"].attention.sinks.grad.abs().sum() > 0
    sd = dict(model.state_dict())
    ad = GptOssStateDictAdapter(cfg, None)
    hf = ad.to_hf(sd)
    assert "model.layers.0.self_attn.sinks" in hf and "model.layers.1.mlp.experts.gate_up_proj_blocks" in hf
    back = ad.from_hf(hf)
    for k, v in sd.items():
        if "expert_bias" in k:
            continue
        assert torch.equal(back[k], v), k


def test_gpt_oss_swiglu_and_mxfp4():
    from torchtitan_b200.models.gpt_oss.moe import swiglu
    from torchtitan_b200.models.gpt_oss.state_dict_adapter import dequantize_mxfp4

    x = torch.tensor([[10.0, 9.0, -1.0, -9.0]])
    out = swiglu(x, limit=7.0)
    exp0 = 7.0 * torch.sigmoid(torch.tensor(1.702 * 7.0)) * (7.0 + 1)
    exp1 = -1.0 * torch.sigmoid(torch.tensor(-1.702)) * (-7.0 + 1)
    assert torch.allclose(out, torch.stack((exp0, exp1)).view(1, 2))
    blocks = torch.zeros(1, 1, 16, dtype=torch.uint8)
    blocks[0, 0, 0] = 0x2 | (0xF << 4)  # values 1.0 and -6.0
    vals = dequantize_mxfp4(blocks, torch.tensor([[128]], dtype=torch.uint8))
    assert vals.shape == (1, 32) and vals[0, 0] == 2.0 and vals[0, 1] == -12.0 and vals[0, 2:].abs().sum() == 0


def test_padded_local_dispatcher_matches_unpadded():
    """The 64-aligned layout (used by the device-side grouped GEMM) gives the same layer output and gradients."""
    from torchtitan_b200.models.common.moe import MoE
    from torchtitan_b200.models.common.moe.moe import LocalDispatcher

    kw = dict(num_experts=8, num_shared_experts=1, score_func="softmax", route_norm=True, top_k=2, hidden_dim=32)
    for before in (True, False):
        torch.manual_seed(0)
        a = MoE.Config(score_before_experts=before, **kw).build(dim=16)
        a.init_weights(init_std=0.02, buffer_device=torch.device("cpu"))
        b = MoE.Config(score_before_experts=before, **kw).build(dim=16)
        b.load_state_dict(a.state_dict())
        b.experts.dispatcher = LocalDispatcher(alignment=64)
        x1 = torch.randn(2, 24, 16, requires_grad=True)
        x2 = x1.detach().clone().requires_grad_()
        ya, yb = a(x1), b(x2)
        ya.square().sum().backward()
        yb.square().sum().backward()
        assert torch.allclose(ya, yb, atol=1e-6)
        assert torch.allclose(x1.grad, x2.grad, atol=1e-6)
        assert torch.allclose(a.experts.w2.grad, b.experts.w2.grad, atol=1e-6)
