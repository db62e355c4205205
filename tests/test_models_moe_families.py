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

    cfg = llama4_configs["debugmodel"]
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
