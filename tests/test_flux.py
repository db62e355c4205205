"""FLUX: latent packing, sampler schedule, model forward/backward, autoencoder shapes, one trainer step on CPU."""

import dataclasses

import torch


def test_pack_unpack_and_position_ids():
    from torchtitan_b200.models.flux.utils import create_position_encoding_for_latents, pack_latents, unpack_latents

    x = torch.randn(2, 16, 8, 12)
    p = pack_latents(x)
    assert p.shape == (2, 24, 64) and torch.equal(unpack_latents(p, 8, 12), x)
    import einops

    assert torch.equal(p, einops.rearrange(x, "b c (h ph) (w pw) -> b (h w) (c ph pw)", ph=2, pw=2))
    ids = create_position_encoding_for_latents(2, 8, 12)
    assert ids.shape == (2, 24, 3) and ids[0, 7].tolist() == [0.0, 1.0, 1.0]


def test_schedule_is_monotone_and_shifted():
    from torchtitan_b200.models.flux.inference.sampling import get_schedule

    s = get_schedule(8, 1024)
    assert s[0] == 1.0 and s[-1] == 0.0 and all(a > b for a, b in zip(s, s[1:]))
    plain = get_schedule(8, 1024, shift=False)
    assert all(a >= b for a, b in zip(s[1:-1], plain[1:-1]))   # the shift spends more steps at high noise


def test_flux_model_and_autoencoder():
    from torchtitan_b200.models.flux import flux_configs
    from torchtitan_b200.models.flux.model.autoencoder import AutoEncoder

    cfg = flux_configs["flux-debug"]
    torch.manual_seed(0)
    model = cfg.build()
    model.init_weights()
    B, L, T = 2, 16, 8
    img, txt = torch.randn(B, L, 64), torch.randn(B, T, cfg.context_in_dim)
    img_ids = torch.zeros(B, L, 3)
    img_ids[..., 1] = torch.arange(L).view(1, L) // 4
    img_ids[..., 2] = torch.arange(L).view(1, L) % 4
    out = model(img=img, img_ids=img_ids, txt=txt, txt_ids=torch.zeros(B, T, 3), timesteps=torch.rand(B), y=torch.randn(B, cfg.vec_in_dim))
    assert out.shape == (B, L, 64)
    assert out.abs().max() == 0          # zero-initialised final layer: the model starts as the zero velocity field
    torch.nn.init.normal_(model.final_layer.linear.weight, std=0.02)
    out = model(img=img, img_ids=img_ids, txt=txt, txt_ids=torch.zeros(B, T, 3), timesteps=torch.rand(B), y=torch.randn(B, cfg.vec_in_dim))
    out.square().mean().backward()
    assert model.double_blocks[0].img_attn.qkv.weight.grad is not None and model.single_blocks[1].linear1.weight.grad is not None
    ae = AutoEncoder(cfg.autoencoder_params)
    x = torch.randn(1, 3, 64, 64)
    z = ae.encode(x)
    assert z.shape == (1, 16, 8, 8) and ae.decode(z).shape == x.shape


def test_flux_trainer_steps_on_cpu(tmp_path, monkeypatch):
    from torchtitan_b200.models.flux.config_registry import flux_debugmodel
    from torchtitan_b200.models.flux.inference.sampling import generate_image, save_image

    monkeypatch.setenv("LOCAL_RANK", "0")
    cfg = flux_debugmodel()
    cfg.dump_folder = str(tmp_path)
    cfg.training.steps, cfg.training.local_batch_size, cfg.training.dtype = 2, 2, "float32"
    cfg.activation_checkpoint.mode = "none"
    cfg.checkpoint.enable = False
    tr = cfg.build()
    it = tr.batch_generator(tr.dataloader) if hasattr(tr, "batch_generator") else iter(tr.dataloader)
    for _ in range(2):
        tr.train_step(it)
        tr.step += 1
    assert float(tr.last_loss) == float(tr.last_loss) and float(tr.last_loss) > 0
    inputs, images = next(iter(tr.dataloader))
    imgs = generate_image(tr.device, tr._dtype, model=tr.model_parts[0], autoencoder=tr.autoencoder, clip_encoder=tr.clip_encoder,
                          t5_encoder=tr.t5_encoder, clip_tokens=inputs["clip_tokens"][:1], t5_tokens=inputs["t5_tokens"][:1],
                          height=64, width=64, steps=2)
    assert imgs.shape == (1, 3, 64, 64)
    path = save_image(imgs[0], str(tmp_path / "img"), "sample.png")
    import os

    assert os.path.getsize(path) > 0
    tr.close()
