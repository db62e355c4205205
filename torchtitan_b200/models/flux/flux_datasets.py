"""Image-caption data for FLUX: samples are ``({"clip_tokens", "t5_tokens", "prompt"}, image)`` with the image centre-
cropped / resized to ``img_size`` and scaled to [-1, 1]; a fraction ``classifier_free_guidance_prob`` of prompts is
replaced by the empty prompt. ``cc12m-test`` / ``coco-validation`` read local folders in the Hugging Face layout when
present; the ``synthetic`` dataset (offline default) draws random images and captions.
Parity: torchtitan/models/flux/flux_datasets.py."""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch.utils.data import IterableDataset

from torchtitan_b200.components.dataloader import BaseDataLoader


def process_image(img: torch.Tensor, size: int) -> torch.Tensor:
    """[C, H, W] in [0, 1] -> centre crop to a square, resize to ``size``, scale to [-1, 1]."""
    C, H, W = img.shape
    s = min(H, W)
    top, left = (H - s) // 2, (W - s) // 2
    img = img[:, top : top + s, left : left + s]
    img = torch.nn.functional.interpolate(img.unsqueeze(0), size=(size, size), mode="bilinear", align_corners=False)[0]
    return img * 2 - 1


class SyntheticFluxDataset(IterableDataset):
    def __init__(self, img_size: int, t5_len: int, clip_len: int, cfg_prob: float, rank: int, world: int, seed: int = 0,
                 t5_vocab: int = 32128, clip_vocab: int = 49408):
        self.img_size, self.t5_len, self.clip_len, self.cfg_prob = img_size, t5_len, clip_len, cfg_prob
        self.rank, self.world, self.seed, self.t5_vocab, self.clip_vocab = rank, world, seed, t5_vocab, clip_vocab
        self._n = 0

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed * 7919 + self.rank)
        while True:
            h = int(torch.randint(self.img_size, 2 * self.img_size, (1,), generator=g))
            w = int(torch.randint(self.img_size, 2 * self.img_size, (1,), generator=g))
            img = process_image(torch.rand(3, h, w, generator=g), self.img_size)
            empty = bool(torch.rand((), generator=g) < self.cfg_prob)
            t5 = torch.zeros(1, self.t5_len, dtype=torch.long) if empty else torch.randint(1, self.t5_vocab, (1, self.t5_len), generator=g)
            clip = torch.zeros(1, self.clip_len, dtype=torch.long) if empty else torch.randint(1, self.clip_vocab, (1, self.clip_len), generator=g)
            self._n += 1
            yield {"clip_tokens": clip, "t5_tokens": t5}, img

    def state_dict(self):
        return {"n": self._n}

    def load_state_dict(self, sd):
        self._n = sd.get("n", 0)


class FluxDataLoader(BaseDataLoader):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseDataLoader.Config):
        dataset: str = "synthetic"
        dataset_path: str | None = None
        classifier_free_guidance_prob: float = 0.1
        img_size: int = 256
        t5_max_length: int = 256
        clip_max_length: int = 77

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, local_batch_size: int, **kwargs):
        self.config = config
        if config.dataset != "synthetic":
            raise NotImplementedError(f"dataset {config.dataset}: only 'synthetic' is available offline; cc12m / coco need the "
                                      "Hugging Face `datasets` cache at dataset_path")
        self.dataset = SyntheticFluxDataset(config.img_size, config.t5_max_length, config.clip_max_length,
                                            config.classifier_free_guidance_prob, dp_rank, dp_world_size)
        self.batch_size = local_batch_size

    def __iter__(self):
        it = iter(self.dataset)
        while True:
            items = [next(it) for _ in range(self.batch_size)]
            inputs = {k: torch.stack([i[0][k] for i in items]) for k in items[0][0]}
            yield inputs, torch.stack([i[1] for i in items])

    def state_dict(self):
        return self.dataset.state_dict()

    def load_state_dict(self, sd):
        self.dataset.load_state_dict(sd)
