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
    cfg = _small_inputs(flux_debugmodel())
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


def _small_inputs(cfg):
    """The debug job at 64 pixels and 16-token prompts: CPU-sized."""
    for dl in (cfg.dataloader, cfg.validator.dataloader):
        dl.img_size, dl.t5_max_length, dl.clip_max_length = 64, 16, 16
    cfg.validator.steps = 2
    return cfg


def _tiny_flux_config(tmp_path):
    from torchtitan_b200.models.flux import model_registry
    from torchtitan_b200.models.flux.config_registry import flux_debugmodel

    cfg = _small_inputs(flux_debugmodel())
    cfg.model_spec = model_registry("flux-debug-tiny")
    cfg.dump_folder = str(tmp_path)
    cfg.training.steps, cfg.training.local_batch_size, cfg.training.dtype = 2, 2, "float32"
    cfg.activation_checkpoint.mode = "none"
    cfg.checkpoint.enable = False
    return cfg


def test_flux_inference_entry_point_and_guided_sampling(tmp_path, monkeypatch):
    """Prompt file -> images through the trainer object, with classifier-free guidance (batched unconditional +
    conditional passes) and the per-rank prompt shares."""
    from PIL import ExifTags, Image

    from torchtitan_b200.models.flux.inference.infer import inference, read_prompts, share_of
    from torchtitan_b200.models.flux.inference.sampling import denoise

    monkeypatch.setenv("LOCAL_RANK", "0")
    assert share_of(7, 0, 3, 2) == ([0, 3, 6], 2) and share_of(7, 2, 3, 2) == ([2, 5], 2)
    assert share_of(5, 3, 4, 2) == ([3], 1) and share_of(9, 3, 4, 2) == ([3, 7], 2)
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("a red cube on a table\n\nan empty street at night\na third prompt\n")
    assert read_prompts(str(prompts)) == ["a red cube on a table", "an empty street at night", "a third prompt"]
    cfg = _tiny_flux_config(tmp_path)
    cfg.inference.prompts_path, cfg.inference.local_batch_size, cfg.inference.img_size = str(prompts), 2, 32
    cfg.validation.denoising_steps, cfg.validation.enable_classifier_free_guidance = 2, True
    cfg.validation.classifier_free_guidance_scale = 3.0
    files = inference(cfg)
    assert [f.rsplit("/", 1)[1] for f in files] == [f"image_prompt{i}_rank0.png" for i in range(3)]
    im = Image.open(files[1])
    assert im.size == (32, 32) and im.getexif()[ExifTags.Base.ImageDescription] == "an empty street at night"

    # the batched guided step equals two separate passes combined by hand
    class Field(torch.nn.Module):
        def forward(self, img, img_ids, txt, txt_ids, y, timesteps):
            return img * y.mean(1).view(-1, 1, 1) + txt.mean((1, 2)).view(-1, 1, 1) * timesteps.view(-1, 1, 1)

    torch.manual_seed(0)
    lat = torch.randn(2, 16, 4, 4)
    clip, t5, eclip, et5 = torch.randn(2, 8), torch.randn(2, 5, 8), torch.randn(2, 8), torch.randn(2, 5, 8)
    got = denoise(Field(), lat, clip, t5, steps=3, cfg_scale=2.5, empty_clip=eclip, empty_t5=et5)
    from torchtitan_b200.models.flux.inference.sampling import get_schedule
    from torchtitan_b200.models.flux.utils import pack_latents, unpack_latents

    x = pack_latents(lat)
    ts = get_schedule(3, x.shape[1])
    f = Field()
    for t_cur, t_prev in zip(ts[:-1], ts[1:]):
        tv = torch.full((2,), t_cur)
        co, un = f(x, None, t5, None, clip, tv), f(x, None, et5, None, eclip, tv)
        x = x + (t_prev - t_cur) * (un + 2.5 * (co - un))
    assert torch.allclose(got, unpack_latents(x, 4, 4), atol=1e-5)
    plain = denoise(Field(), lat, clip, t5, steps=3)
    assert not torch.allclose(plain, got)


def test_flux_validator_samples_prompts_and_noise_differs_by_rank(tmp_path, monkeypatch):
    import dataclasses
    import os

    from torchtitan_b200.models.flux.flux_datasets import FluxDataLoader

    monkeypatch.setenv("LOCAL_RANK", "0")
    folder, _ = _make_image_data(tmp_path)
    cfg = _tiny_flux_config(tmp_path)
    cfg.validation.denoising_steps = 1
    cfg.validator = dataclasses.replace(
        cfg.validator, enable=True, steps=2, all_timesteps=False, save_img_count=3, save_img_folder="validation_images",
        dataloader=FluxDataLoader.Config(dataset="coco-validation", dataset_path=str(folder), img_size=32, t5_max_length=16,
                                         clip_max_length=16, classifier_free_guidance_prob=0.0, test_tokenizer=True))
    tr = cfg.build()
    assert tr.validator.dataloader.config.generate_timesteps            # round-robin noise levels come from the loader
    loss = tr.validator.validate(tr.model_parts, step=7)
    assert loss == loss and loss > 0
    saved = sorted(os.listdir(os.path.join(str(tmp_path), "validation_images")))
    assert saved == [f"image_rank0_7_{i}.png" for i in range(3)]       # 2 from the first batch, 1 from the second
    # the trainer's noise stream depends on the data-parallel rank and on the base seed only
    g0 = tr._noise_gen.initial_seed()
    assert g0 == (tr.base_seed + 1_000_003 * (tr.dp_rank + 1)) % 2**63
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
        arr = (np.random.RandomState(i).rand(40 + 3 * i, 56, 3) * 255).astype("uint8")     # all at least 32 pixels on a side
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
    assert [b[1].shape[0] for b in batches] == [2, 2, 2, 1]              # 7 readable images in batches of 2
    inp, img = batches[0]
    assert img.shape == (2, 3, 32, 32) and float(img.min()) >= -1 and float(img.max()) <= 1
    assert inp["t5_tokens"].shape == (2, 16) and inp["clip_tokens"].shape == (2, 8)
    assert inp["prompt"] == ["a picture number 0", "a picture number 1"]
    # web-dataset shards, split over two data-parallel ranks by shard
    r0 = [p for b in loader("cc12m-wds", wds, 0, 2) for p in b[0]["prompt"]]
    r1 = [p for b in loader("cc12m-wds", wds, 1, 2) for p in b[0]["prompt"]]
    assert r0 == ["caption 0", "caption 2", "caption 4", "caption 6"] and r1 == ["caption 1", "caption 3", "caption 5"]
    # resume: the state counts consumed samples
    dl = loader("cc12m-test", folder)
    it = iter(dl)
    next(it)
    state = dl.state_dict()
    want = next(it)[0]["prompt"]
    dl2 = loader("cc12m-test", folder)
    dl2.load_state_dict(state)
    assert next(iter(dl2))[0]["prompt"] == want
    # classifier-free guidance replaces the token rows by those of the empty prompt, each encoder on its own draw
    def guided(p):
        return FluxDataLoader(FluxDataLoader.Config(dataset="cc12m-test", dataset_path=str(folder), img_size=32, t5_max_length=16,
                                                    clip_max_length=8, classifier_free_guidance_prob=p, test_tokenizer=True,
                                                    infinite=False), dp_world_size=1, dp_rank=0, local_batch_size=1)
    empty_t5, empty_clip = FluxTestTokenizer(16, 32128).encode("")[0], FluxTestTokenizer(8, 49408).encode("")[0]
    dropped = list(guided(1.0))
    assert dropped and all(torch.equal(b[0]["t5_tokens"][0], empty_t5) and torch.equal(b[0]["clip_tokens"][0], empty_clip)
                           for b in dropped)
    assert [b[0]["prompt"] for b in dropped] == [[f"a picture number {i}"] for i in range(7)]      # the prompt itself stays
    half = list(guided(0.5))
    kinds = {(bool(torch.equal(b[0]["t5_tokens"][0], empty_t5)), bool(torch.equal(b[0]["clip_tokens"][0], empty_clip))) for b in half}
    assert len(kinds) >= 2                                                # independent draws: not always both or neither
    # exact resume, random crops and guidance draws included
    a = guided(0.5)
    it = iter(a)
    next(it), next(it)
    state = a.state_dict()
    rest = list(it)
    b = guided(0.5)
    b.load_state_dict(state)
    again = list(b)
    assert len(rest) == len(again) == 5
    for (i1, l1), (i2, l2) in zip(rest, again):
        assert torch.equal(l1, l2) and torch.equal(i1["t5_tokens"], i2["t5_tokens"]) and torch.equal(i1["clip_tokens"], i2["clip_tokens"])
    # validation loaders attach the eight stratified noise levels in turn
    val = FluxDataLoader(FluxDataLoader.Config(dataset="coco-validation", dataset_path=str(folder), img_size=32, t5_max_length=16,
                                               clip_max_length=8, classifier_free_guidance_prob=0.0, test_tokenizer=True,
                                               infinite=False, generate_timesteps=True), dp_world_size=1, dp_rank=0, local_batch_size=2)
    ts = torch.cat([b[0]["timestep"] for b in val])
    assert torch.allclose(ts, torch.tensor([(i + 0.5) / 8 for i in range(7)]))
    # loader workers: decoding runs in two worker processes that share the rank's samples between them
    w2 = FluxDataLoader(FluxDataLoader.Config(dataset="cc12m-test", dataset_path=str(folder), img_size=32, t5_max_length=16,
                                              clip_max_length=8, classifier_free_guidance_prob=0.0, test_tokenizer=True,
                                              infinite=False, num_workers=2), dp_world_size=1, dp_rank=0, local_batch_size=1)
    assert sorted(b[0]["prompt"][0] for b in w2) == [f"a picture number {i}" for i in range(7)]
    # images smaller than the target are skipped
    small = FluxDataLoader(FluxDataLoader.Config(dataset="cc12m-test", dataset_path=str(folder), img_size=48, t5_max_length=16,
                                                 clip_max_length=8, classifier_free_guidance_prob=0.0, test_tokenizer=True,
                                                 infinite=False), dp_world_size=1, dp_rank=0, local_batch_size=1)
    assert [b[0]["prompt"][0] for b in small] == [f"a picture number {i}" for i in range(3, 7)]     # heights 40 + 3 i >= 48
    # the registry is open: a user entry with its own loader and a processor of the reference's signature
    from torchtitan_b200.hf_datasets import DatasetConfig
    from torchtitan_b200.models.flux import flux_datasets as fd

    class Mine(fd.LocalSamples):
        def __init__(self, path, kind="mine", rank=0, world=1):
            super().__init__(path, kind, rank, world)

        def shard(self, rank, world):
            return Mine(self.path, "mine", rank, world)

        def __iter__(self):
            from PIL import Image

            for i in range(6):
                if i % self.world == self.rank:
                    yield {"picture": Image.new("L", (64, 40 + i), color=10 * i), "words": f"mine {i}"}

    def mine_processor(sample, t5_tokenizer, clip_tokenizer, output_size=256):
        return fd._cc12m_wds_data_processor({"jpg": sample["picture"], "txt": sample["words"]}, t5_tokenizer, clip_tokenizer, output_size)

    fd.DATASETS["mine"] = DatasetConfig(path=str(tmp_path), loader=Mine, sample_processor=mine_processor)
    try:
        got = [p for b in loader("mine", tmp_path, 1, 2) for p in b[0]["prompt"]]
        assert got == ["mine 1", "mine 3", "mine 5"]                     # rank 1 of 2, grey images become RGB
    finally:
        del fd.DATASETS["mine"]
    import pytest

    with pytest.raises(ValueError, match="is not supported"):
        loader("no-such-dataset", folder)
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
