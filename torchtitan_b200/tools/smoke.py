"""One tiny Llama-3 training step on cuda:0 through the native kernels (used by the build's
smoke check and by the GPU tests)."""

from __future__ import annotations

import torch


def tiny_llama_config(seq_len: int = 256):
    from torchtitan_b200.models.common import Embedding, FeedForward, GQAttention, Linear, RMSNorm, RoPE
    from torchtitan_b200.models.llama3 import Llama3Model, Llama3TransformerBlock

    return Llama3Model.Config(
        dim=512, n_layers=2, vocab_size=4096,
        tok_embeddings=Embedding.Config(), norm=RMSNorm.Config(), output=Linear.Config(),
        layer=Llama3TransformerBlock.Config(
            attention_norm=RMSNorm.Config(), ffn_norm=RMSNorm.Config(),
            feed_forward=FeedForward.Config(hidden_dim=1536),
            attention=GQAttention.Config(n_heads=4, n_kv_heads=2, attn_backend="sdpa", rope_backend="complex"),
        ),
        rope=RoPE.Config(dim=128, max_seq_len=seq_len, theta=500000, backend="complex", scaling="llama"),
    )


def run_smoke(steps: int = 2, seq_len: int = 256, batch: int = 2) -> float:
    from torchtitan_b200.components.loss import cross_entropy_loss
    from torchtitan_b200.components.optimizer import OptimizersContainer
    from torchtitan_b200.ops import native
    from torchtitan_b200.parallel import fsdp
    from torchtitan_b200.parallel.data_parallel import apply_single_device_units

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    cfg = tiny_llama_config(seq_len)
    with torch.device("meta"):
        model = cfg.build()
    apply_single_device_units(model, param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    model.to_empty(device=dev)
    with torch.no_grad():
        model.init_weights()
    fsdp.materialize(model)
    opt = OptimizersContainer.Config(lr=1e-3).build(model_parts=[model])
    loss_val = None
    for _ in range(steps):
        tokens = torch.randint(0, cfg.vocab_size, (batch, seq_len + 1), device=dev)
        opt.zero_grad()
        logits = model(tokens[:, :-1])
        loss = cross_entropy_loss(logits, tokens[:, 1:]) / (batch * seq_len)
        loss.backward()
        opt.step()
        loss_val = float(loss)
    torch.cuda.synchronize()
    errs = native.kernel_errors()
    assert not errs, f"kernel error flags: {errs}"
    assert loss_val == loss_val and loss_val < 20.0, f"bad loss {loss_val}"
    return loss_val
