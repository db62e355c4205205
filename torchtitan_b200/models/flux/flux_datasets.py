"""Image-caption data for FLUX: samples are ``({"clip_tokens", "t5_tokens", "prompt"}, image)`` with the image centre-
cropped / resized to ``img_size`` and scaled to [-1, 1]; a fraction ``classifier_free_guidance_prob`` of prompts is
replaced by the empty prompt. The ``synthetic`` dataset (offline default) draws random images and captions; the named
image-caption datasets read local copies at ``dataset_path``:

* ``cc12m-wds``: webdataset shards (``*.tar`` holding ``<key>.jpg|png|webp`` + ``<key>.txt``), streamed shard by shard;
* ``cc12m-test`` / ``coco-validation`` (and any other name): an image folder with ``metadata.jsonl`` lines
  ``{"file_name": ..., "text" | "caption": ...}`` (COCO's list of captions uses the first one).

Shards / rows are dealt round-robin to data-parallel ranks; the state is the number of samples consumed, so a resumed
loader skips to where it stopped. Undecodable or tiny images are skipped.
Parity: torchtitan/models/flux/flux_datasets.py (dataset registry, ``_cc12m_wds_data_processor``,
``_coco_data_processor``, FluxDataset / FluxValidationDataset)."""

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


def _decode_image(data) -> torch.Tensor | None:
    """bytes / path -> float [3, H, W] in [0, 1], or None when the file is not a usable image."""
    import io

    import numpy as np
    from PIL import Image

    try:
        im = Image.open(io.BytesIO(data) if isinstance(data, (bytes, bytearray)) else data).convert("RGB")
    except Exception:
        return None
    if min(im.size) < 8:
        return None
    return torch.from_numpy(np.asarray(im, dtype=np.uint8).copy()).permute(2, 0, 1).float() / 255.0


def _iter_folder(path: str):
    import json
    import os

    with open(os.path.join(path, "metadata.jsonl")) as f:
        for line in f:
            if not line.strip():
                continue
            row = json.loads(line)
            text = row.get("text", row.get("caption", row.get("captions", "")))
            if isinstance(text, (list, tuple)):
                text = text[0] if text else ""
            yield os.path.join(path, row["file_name"]), str(text)


def _iter_wds(path: str, rank: int, world: int):
    import glob
    import os
    import tarfile

    shards = sorted(glob.glob(os.path.join(path, "*.tar")))
    if not shards:
        raise FileNotFoundError(f"no *.tar shards under {path}")
    for shard in shards[rank::world] if len(shards) >= world else shards:
        with tarfile.open(shard) as tar:
            pending: dict[str, dict] = {}
            for m in tar:
                if not m.isfile():
                    continue
                key, ext = os.path.splitext(m.name)
                ext = ext.lower().lstrip(".")
                slot = pending.setdefault(key, {})
                slot["txt" if ext == "txt" else "img"] = tar.extractfile(m).read()
                if "txt" in slot and "img" in slot:
                    yield slot["img"], slot["txt"].decode("utf-8", "replace").strip()
                    del pending[key]


class ImageCaptionDataset(IterableDataset):
    """Named image-caption dataset read from a local copy (see the module docstring)."""

    def __init__(self, name: str, path: str, t5_tokenizer, clip_tokenizer, img_size: int, cfg_prob: float, rank: int,
                 world: int, infinite: bool = True, seed: int = 0):
        import os

        if path is None or not os.path.isdir(path):
            raise FileNotFoundError(f"dataset {name}: local copy not found at dataset_path={path!r}")
        self.name, self.path, self.t5, self.clip = name, path, t5_tokenizer, clip_tokenizer
        self.img_size, self.cfg_prob, self.rank, self.world = img_size, cfg_prob, rank, world
        self.infinite, self.seed = infinite, seed
        self._consumed = 0
        self._wds = name.endswith("-wds") or not os.path.exists(os.path.join(path, "metadata.jsonl"))

    def _rows(self):
        import glob
        import os

        if self._wds:
            sharded = len(glob.glob(os.path.join(self.path, "*.tar"))) >= self.world
            for i, item in enumerate(_iter_wds(self.path, self.rank, self.world)):
                if sharded or i % self.world == self.rank:
                    yield item
        else:
            for i, item in enumerate(_iter_folder(self.path)):
                if i % self.world == self.rank:
                    yield item

    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed * 7919 + self.rank)
        skip = self._consumed
        while True:
            n = 0
            for src, text in self._rows():
                n += 1
                if skip > 0:
                    skip -= 1
                    torch.rand((), generator=g)                # keep the guidance draws aligned with the first pass
                    continue
                drop = bool(torch.rand((), generator=g) < self.cfg_prob)
                self._consumed += 1
                img = _decode_image(src)
                if img is None:
                    continue
                prompt = "" if drop else text
                yield {"clip_tokens": self.clip.encode(prompt), "t5_tokens": self.t5.encode(prompt), "prompt": prompt}, \
                    process_image(img, self.img_size)
            if not self.infinite or n == 0:
                return

    def state_dict(self):
        return {"consumed": self._consumed}

    def load_state_dict(self, sd):
        self._consumed = int(sd.get("consumed", 0))


DATASETS = ("synthetic", "cc12m-wds", "cc12m-test", "coco-validation")


class FluxDataLoader(BaseDataLoader):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseDataLoader.Config):
        dataset: str = "synthetic"
        dataset_path: str | None = None
        classifier_free_guidance_prob: float = 0.1
        img_size: int = 256
        t5_max_length: int = 256
        clip_max_length: int = 77
        t5_tokenizer_path: str | None = None
        clip_tokenizer_path: str | None = None
        test_tokenizer: bool = False
        """Use the asset-free tokenizer (also chosen when the tokenizer folders are missing)."""
        infinite: bool = True

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, local_batch_size: int, **kwargs):
        self.config = config
        if config.dataset == "synthetic":
            self.dataset = SyntheticFluxDataset(config.img_size, config.t5_max_length, config.clip_max_length,
                                                config.classifier_free_guidance_prob, dp_rank, dp_world_size)
        else:
            from .tokenizer import build_flux_tokenizer

            t5, clip = build_flux_tokenizer(t5_path=config.t5_tokenizer_path, clip_path=config.clip_tokenizer_path,
                                            t5_max_length=config.t5_max_length, clip_max_length=config.clip_max_length,
                                            test_mode=config.test_tokenizer)
            self.dataset = ImageCaptionDataset(config.dataset, config.dataset_path, t5, clip, config.img_size,
                                               config.classifier_free_guidance_prob, dp_rank, dp_world_size,
                                               infinite=config.infinite)
        self.batch_size = local_batch_size

    def __iter__(self):
        it = iter(self.dataset)
        while True:
            items = []
            for _ in range(self.batch_size):
                try:
                    items.append(next(it))
                except StopIteration:
                    return
            inputs = {k: (torch.stack([i[0][k] for i in items]) if torch.is_tensor(items[0][0][k]) else [i[0][k] for i in items])
                      for k in items[0][0]}
            yield inputs, torch.stack([i[1] for i in items])

    def state_dict(self):
        return self.dataset.state_dict()

    def load_state_dict(self, sd):
        self.dataset.load_state_dict(sd)
