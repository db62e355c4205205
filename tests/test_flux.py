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


def _make_image_data(root, n=7):
    import io
    import json
    import tarfile

    import numpy as np
    from PIL import Image

    folder, wds = root / "folder", root / "wds"
    folder.mkdir()
    wds.mkdir()
    rows = []
    tars = [tarfile.open(wds / f"shard-{i:03d}.tar", "w") for i in range(2)]
    for i in range(n):
        arr = (np.random.RandomState(i).rand(40 + 3 * i, 56, 3) * 255).astype("uint8")
        im = Image.fromarray(arr)
        im.save(folder / f"img{i}.png")
        rows.append({"file_name": f"img{i}.png", "captions" if i % 2 else "text": [f"a picture number {i}"] if i % 2 else f"a picture number {i}"})
        buf = io.BytesIO()
        im.save(buf, format="JPEG")
        for name, data in ((f"{i:05d}.jpg", buf.getvalue()), (f"{i:05d}.txt", f"caption {i}".encode())):
            info = tarfile.TarInfo(name)
            info.size = len(data)
            tars[i % 2].addfile(info, io.BytesIO(data))
    (folder / "broken.png").write_bytes(b"not an image")
    rows.append({"file_name": "broken.png", "text": "unreadable"})
    with open(folder / "metadata.jsonl", "w") as f:
        f.write("\n".join(json.dumps(r) for r in rows))
    for t in tars:
        t.close()
    return folder, wds


def test_image_caption_datasets_folder_and_webdataset(tmp_path):
    from torchtitan_b200.models.flux.flux_datasets import FluxDataLoader
    from torchtitan_b200.models.flux.tokenizer import FluxTestTokenizer, build_flux_tokenizer

    folder, wds = _make_image_data(tmp_path)
    tok = FluxTestTokenizer(max_length=8, vocab_size=100)
    ids = tok.encode(["a b c", ""])
    assert ids.shape == (2, 8) and ids[0, 3] == 99 and ids[1, 0] == 99 and (ids[1, 1:] == 0).all()
    assert torch.equal(tok.encode("a b c"), ids[:1])
    t5, clip = build_flux_tokenizer(t5_path=None, clip_path=str(tmp_path / "missing"), t5_max_length=16, clip_max_length=8)
    assert t5.encode("x").shape == (1, 16) and clip.encode("x").shape == (1, 8)

    def loader(name, path, rank=0, world=1, **kw):
        cfg = FluxDataLoader.Config(dataset=name, dataset_path=str(path), img_size=32, t5_max_length=16, clip_max_length=8,
                                    classifier_free_guidance_prob=0.0, test_tokenizer=True, infinite=False, **kw)
        return FluxDataLoader(cfg, dp_world_size=world, dp_rank=rank, local_batch_size=2)

    batches = list(loader("coco-validation", folder))
    assert len(batches) == 3                                             # 7 readable images -> 3 full batches of 2
    inp, img = batches[0]
    assert img.shape == (2, 3, 32, 32) and float(img.min()) >= -1 and float(img.max()) <= 1
    assert inp["t5_tokens"].shape == (2, 1, 16) and inp["clip_tokens"].shape == (2, 1, 8)
    assert inp["prompt"] == ["a picture number 0", "a picture number 1"]
    # web-dataset shards, split over two data-parallel ranks by shard
    r0 = [p for b in loader("cc12m-wds", wds, 0, 2) for p in b[0]["prompt"]]
    r1 = [p for b in loader("cc12m-wds", wds, 1, 2) for p in b[0]["prompt"]]
    assert r0 == ["caption 0", "caption 2", "caption 4", "caption 6"] and r1 == ["caption 1", "caption 3"]
    # resume: the state counts consumed samples
    dl = loader("cc12m-test", folder)
    it = iter(dl)
    next(it)
    state = dl.state_dict()
    want = next(it)[0]["prompt"]
    dl2 = loader("cc12m-test", folder)
    dl2.load_state_dict(state)
    assert next(iter(dl2))[0]["prompt"] == want
    # classifier-free guidance drops prompts
    dropped = [p for b in loader("cc12m-test", folder).__class__(
        FluxDataLoader.Config(dataset="cc12m-test", dataset_path=str(folder), img_size=32, t5_max_length=16, clip_max_length=8,
                              classifier_free_guidance_prob=1.0, test_tokenizer=True, infinite=False),
        dp_world_size=1, dp_rank=0, local_batch_size=1) for p in b[0]["prompt"]]
    assert dropped and all(p == "" for p in dropped)
    import pytest

    with pytest.raises(FileNotFoundError):
        loader("cc12m-test", tmp_path / "nowhere")


def test_flux_hf_adapter_splits_fused_projections_and_round_trips():
    from torchtitan_b200.models.flux.config_registry import flux_debugmodel
    from torchtitan_b200.models.flux.model.state_dict_adapter import FluxStateDictAdapter

    cfg = flux_debugmodel().model_spec.model
    model = cfg.build()
    sd = {k: torch.randn_like(v) for k, v in model.state_dict().items()}
    ad = FluxStateDictAdapter(cfg, None)
    hf = ad.to_hf(sd)
    h = cfg.hidden_size
    assert hf["transformer_blocks.0.attn.to_k.weight"].shape == (h, h)
    assert torch.equal(hf["transformer_blocks.0.attn.to_k.weight"], sd["double_blocks.0.img_attn.qkv.weight"][h : 2 * h])
    assert torch.equal(hf["transformer_blocks.1.attn.add_v_proj.bias"], sd["double_blocks.1.txt_attn.qkv.bias"][2 * h :])
    assert torch.equal(hf["single_transformer_blocks.0.proj_mlp.weight"], sd["single_blocks.0.linear1.weight"][3 * h :])
    # the final modulation stores (shift, scale) here and (scale, shift) there
    w = sd["final_layer.adaLN_modulation.1.weight"]
    assert torch.equal(hf["norm_out.linear.weight"], torch.cat((w[h:], w[:h])))
    assert "x_embedder.weight" in hf and "time_text_embed.timestep_embedder.linear_1.bias" in hf
    back = ad.from_hf(hf)
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    import pytest

    with pytest.raises(KeyError):
        ad.from_hf({"transformer_blocks.0.attn.to_q.weight": torch.zeros(h, h)})
    with pytest.raises(KeyError):
        ad.to_hf({"unknown.weight": torch.zeros(1)})
