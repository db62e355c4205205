"""Image-caption data for FLUX.

A sample is ``({"clip_tokens", "t5_tokens", "prompt"}, image)``: the image resized so that its short side equals
``img_size``, cropped to a square at a random offset along the long side and scaled to [-1, 1]; images smaller than
``img_size`` are skipped. With probability ``classifier_free_guidance_prob`` the T5 tokens, and independently the CLIP
tokens, are replaced by those of the empty prompt.

``DATASETS`` is a registry of ``DatasetConfig(path, loader, sample_processor)`` entries that users extend
(torchtitan/models/flux/flux_datasets.py:80-173: ``cc12m-wds``, ``cc12m-test``, ``coco-validation``, the two sample
processors and the name check). ``loader(path)`` returns the raw samples: a Hugging Face ``Dataset`` /
``IterableDataset`` (split over data-parallel ranks with ``split_dataset_by_node``, resumed through its own state), or
any object with ``shard(rank, world)`` and ``__iter__`` such as :class:`LocalSamples`, which the built-in loaders return
for a local copy so that neither the ``datasets`` library nor a network is needed:

* a folder of WebDataset shards (``*.tar`` holding ``<key>.jpg|png|webp`` + ``<key>.txt``), dealt shard by shard to the
  ranks when there are at least as many shards as ranks, sample by sample otherwise;
* an image folder with ``metadata.jsonl`` lines ``{"file_name": ..., "text" | "caption" | "captions": ...}``.

A path that is not a local folder goes to ``datasets.load_dataset`` (streaming) as in the reference.

Different from the reference: the random crop and the guidance draws come from a generator owned by the dataset whose
state is part of ``state_dict()``, so a resumed loader continues with exactly the samples the original would have
produced (the reference draws from the global generator); undecodable images are skipped with a warning instead of
ending the job. The ``synthetic`` dataset (random images and token ids) needs no files at all.
"""

from __future__ import annotations

import itertools
import math
import os
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch.utils.data import IterableDataset

from torchtitan_b200.components.dataloader import ParallelAwareDataloader
from torchtitan_b200.hf_datasets import DatasetConfig
from torchtitan_b200.tools.logging import logger

from .configs import Encoder

__all__ = ["DATASETS", "FluxDataset", "FluxValidationDataset", "FluxDataLoader", "LocalSamples", "SyntheticFluxDataset",
           "process_image"]


# ------------------------------------------------------------------------------------------ images
def process_image(img: torch.Tensor, size: int) -> torch.Tensor:
    """[C, H, W] in [0, 1] -> centre crop to a square, resize to ``size``, scale to [-1, 1]."""
    C, H, W = img.shape
    s = min(H, W)
    top, left = (H - s) // 2, (W - s) // 2
    img = img[:, top : top + s, left : left + s]
    img = torch.nn.functional.interpolate(img.unsqueeze(0), size=(size, size), mode="bilinear", align_corners=False)[0]
    return img * 2 - 1


def _open_image(raw):
    """bytes / ``{"bytes": ...}`` / path / PIL image -> PIL image, or None when it cannot be decoded."""
    import io

    from PIL import Image

    try:
        if isinstance(raw, dict):
            raw = raw.get("bytes") or raw.get("path")
        if isinstance(raw, (bytes, bytearray)):
            raw = Image.open(io.BytesIO(raw))
        elif isinstance(raw, (str, os.PathLike)):
            raw = Image.open(raw)
        raw.load()
        return raw
    except Exception as e:
        logger.warning(f"cannot decode image: {type(e).__name__}: {e}")
        return None


def _process_cc12m_image(img, output_size: int = 256, generator: torch.Generator | None = None) -> torch.Tensor | None:
    """Short side to ``output_size``, random square crop along the long side, RGB, [-1, 1]; None for an image that is
    unreadable or smaller than ``output_size`` (torchtitan/models/flux/flux_datasets.py:28-77)."""
    import numpy as np

    img = _open_image(img)
    if img is None:
        return None
    width, height = img.size
    if width < output_size or height < output_size:
        return None
    if width >= height:
        new_w, new_h = math.ceil(output_size / height * width), output_size
        off = int(torch.randint(0, new_w - output_size + 1, (1,), generator=generator))
        box = (off, 0, off + output_size, output_size)
    else:
        new_w, new_h = output_size, math.ceil(output_size / width * height)
        off = int(torch.randint(0, new_h - output_size + 1, (1,), generator=generator))
        box = (0, off, output_size, off + output_size)
    img = img.resize((new_w, new_h)).crop(box)
    if img.mode != "RGB":
        img = img.convert("RGB")
    return torch.from_numpy(np.asarray(img, dtype=np.uint8).copy()).permute(2, 0, 1).float() / 255.0 * 2.0 - 1.0


def _cc12m_wds_data_processor(sample: dict[str, Any], t5_tokenizer, clip_tokenizer, output_size: int = 256,
                              generator: torch.Generator | None = None) -> dict[str, Any]:
    """WebDataset sample ``{"jpg": image, "txt": caption}`` -> image tensor (or None) and the two token rows."""
    text = sample["txt"]
    if isinstance(text, (bytes, bytearray)):
        text = text.decode("utf-8", "replace").strip()
    return {"image": _process_cc12m_image(sample["jpg"], output_size, generator),
            "clip_tokens": clip_tokenizer.encode(text), "t5_tokens": t5_tokenizer.encode(text), "prompt": text}


def _coco_data_processor(sample: dict[str, Any], t5_tokenizer, clip_tokenizer, output_size: int = 256,
                         generator: torch.Generator | None = None) -> dict[str, Any]:
    """COCO sample ``{"image": image, "caption": text or list of texts}``; the first caption is used."""
    text = sample["caption"]
    if isinstance(text, (list, tuple)):
        text = text[0] if text else ""
    return {"image": _process_cc12m_image(sample["image"], output_size, generator),
            "clip_tokens": clip_tokenizer.encode(text), "t5_tokens": t5_tokenizer.encode(text), "prompt": str(text)}


def _call_processor(fn, sample, t5, clip, size, generator):
    """Sample processors registered by users may have the reference's four-argument signature."""
    try:
        return fn(sample, t5, clip, output_size=size, generator=generator)
    except TypeError as e:
        if "generator" not in str(e):
            raise
        return fn(sample, t5, clip, output_size=size)


# ------------------------------------------------------------------------------------------ local readers
class LocalSamples:
    """Raw samples of a local dataset copy. ``kind`` is ``"wds"`` (a folder of tar shards, samples
    ``{"__key__", "jpg", "txt"}``) or ``"folder"`` (``metadata.jsonl`` beside the images, samples
    ``{"__key__", "image": path, "caption"}`` and the same under ``jpg`` / ``txt``)."""

    def __init__(self, path: str, kind: str, rank: int = 0, world: int = 1):
        self.path, self.kind, self.rank, self.world = path, kind, rank, world

    def shard(self, rank: int, world: int) -> "LocalSamples":
        return LocalSamples(self.path, self.kind, rank, world)

    def _wds(self):
        import glob
        import tarfile

        shards = sorted(glob.glob(os.path.join(self.path, "*.tar")))
        if not shards:
            raise FileNotFoundError(f"no *.tar shards under {self.path}")
        by_shard = len(shards) >= self.world
        index = 0
        for shard in shards[self.rank :: self.world] if by_shard else shards:
            with tarfile.open(shard) as tar:
                pending: dict[str, dict] = {}
                for m in tar:
                    if not m.isfile():
                        continue
                    key, ext = os.path.splitext(m.name)
                    ext = ext.lower().lstrip(".")
                    if ext not in ("txt", "jpg", "jpeg", "png", "webp"):
                        continue
                    slot = pending.setdefault(key, {"__key__": key})
                    slot["txt" if ext == "txt" else "jpg"] = tar.extractfile(m).read()
                    if "txt" in slot and "jpg" in slot:
                        del pending[key]
                        if by_shard or index % self.world == self.rank:
                            slot["txt"] = slot["txt"].decode("utf-8", "replace").strip()
                            yield slot
                        index += 1

    def _folder(self):
        import json

        with open(os.path.join(self.path, "metadata.jsonl")) as f:
            rows = [json.loads(line) for line in f if line.strip()]
        for i, row in enumerate(rows):
            if i % self.world != self.rank:
                continue
            text = row.get("text", row.get("caption", row.get("captions", "")))
            if isinstance(text, (list, tuple)):
                text = text[0] if text else ""
            file = os.path.join(self.path, row["file_name"])
            yield {"__key__": row["file_name"], "image": file, "caption": str(text), "jpg": file, "txt": str(text)}

    def __iter__(self):
        return self._wds() if self.kind == "wds" else self._folder()


def _local_kind(path: str) -> str | None:
    if not os.path.isdir(path):
        return None
    return "folder" if os.path.exists(os.path.join(path, "metadata.jsonl")) else "wds"


def _load_train(path: str):
    kind = _local_kind(path)
    if kind is not None:
        return LocalSamples(path, kind)
    from datasets import load_dataset

    return load_dataset(path, split="train", streaming=True)


def _load_validation(path: str):
    kind = _local_kind(path)
    if kind is not None:
        return LocalSamples(path, kind)
    from datasets import load_dataset

    return load_dataset(path, split="validation", streaming=True)


DATASETS: dict[str, DatasetConfig] = {
    "cc12m-wds": DatasetConfig(path="pixparse/cc12m-wds", loader=_load_train, sample_processor=_cc12m_wds_data_processor),
    "cc12m-test": DatasetConfig(path="tests/assets/cc12m_test", loader=_load_train, sample_processor=_cc12m_wds_data_processor),
    "coco-validation": DatasetConfig(path="howard-hou/COCO-Text", loader=_load_validation, sample_processor=_coco_data_processor),
}


def _validate_dataset(dataset_name: str, dataset_path: str | None = None) -> tuple[str, Callable, Callable]:
    if dataset_name not in DATASETS:
        raise ValueError(f"Dataset {dataset_name} is not supported. Supported datasets are: {list(DATASETS.keys())}")
    config = DATASETS[dataset_name]
    path = dataset_path or config.path
    logger.info(f"Preparing {dataset_name} dataset from {path}")
    return path, config.loader, config.sample_processor


# ------------------------------------------------------------------------------------------ datasets
def _worker() -> tuple[int, int]:
    """(index, count) of the loader worker process this code runs in; (0, 1) in the main process."""
    info = torch.utils.data.get_worker_info()
    return (info.id, info.num_workers) if info is not None else (0, 1)


class FluxDataset(IterableDataset):
    """This data-parallel rank's share of a registered image-caption dataset, processed for FLUX."""

    def __init__(self, dataset_name: str, dataset_path: str | None, t5_tokenizer, clip_tokenizer,
                 classifier_free_guidance_prob: float, img_size: int, dp_rank: int = 0, dp_world_size: int = 1,
                 infinite: bool = False, seed: int = 0) -> None:
        dataset_name = dataset_name.lower()
        path, loader, self._data_processor = _validate_dataset(dataset_name, dataset_path)
        if not os.path.isdir(path) and (os.path.isabs(path) or path.startswith(".")):
            raise FileNotFoundError(f"dataset {dataset_name}: local copy not found at {path!r}")
        data = loader(path)
        if isinstance(data, LocalSamples):
            self._data = data.shard(dp_rank, dp_world_size)
        else:
            from datasets.distributed import split_dataset_by_node

            self._data = split_dataset_by_node(data, dp_rank, dp_world_size)
        self.dataset_name = dataset_name
        self._t5, self._clip = t5_tokenizer, clip_tokenizer
        self._t5_empty, self._clip_empty = t5_tokenizer.encode(""), clip_tokenizer.encode("")
        self.classifier_free_guidance_prob, self.img_size, self.infinite = classifier_free_guidance_prob, img_size, infinite
        self._seed = seed * 7919 + dp_rank
        self._gen = torch.Generator().manual_seed(self._seed)
        self._sample_idx = 0                                   # raw samples consumed in the current pass
        self._restored = self._in_worker = False

    def _own_state(self) -> bool:
        """Hugging Face iterable datasets resume through their own ``state_dict``; everything else by skipping."""
        return not isinstance(self._data, LocalSamples) and hasattr(self._data, "state_dict") \
            and hasattr(self._data, "load_state_dict") and not hasattr(self._data, "__len__")

    def _raw(self):
        if self._own_state():
            return iter(self._data)
        if hasattr(self._data, "skip") and hasattr(self._data, "__len__"):            # map-style Hugging Face dataset
            return iter(self._data.skip(self._sample_idx)) if self._sample_idx < len(self._data) else iter(())
        return itertools.islice(iter(self._data), self._sample_idx, None)

    def _enter_worker(self) -> None:
        """First iteration inside a loader worker: this copy of the dataset keeps every k-th local sample (Hugging Face
        datasets deal their shards to the workers themselves) and draws from its own random stream."""
        wid, workers = _worker()
        if workers == 1 or self._in_worker:
            return
        self._in_worker = True
        if isinstance(self._data, LocalSamples):
            d = self._data
            self._data = d.shard(d.rank * workers + wid, d.world * workers)
        if not self._restored:
            self._gen.manual_seed(self._seed * 1_000_003 + wid + 1)

    def __iter__(self):
        self._enter_worker()
        it = self._raw()
        while True:
            sample = next(it, None)
            if sample is None:
                if not self.infinite:
                    logger.warning(f"Dataset {self.dataset_name} has run out of data. "
                                   "This might cause NCCL timeout if data parallelism is enabled.")
                    return
                if self._sample_idx == 0 and not self._own_state():
                    return                                     # an empty share would loop forever
                self._sample_idx = 0
                logger.warning(f"Dataset {self.dataset_name} is being re-looped.")
                if hasattr(self._data, "set_epoch") and hasattr(self._data, "epoch"):
                    self._data.set_epoch(self._data.epoch + 1)
                it = self._raw()
                continue
            self._sample_idx += 1
            out = _call_processor(self._data_processor, sample, self._t5, self._clip, self.img_size, self._gen)
            if out["image"] is None:
                key = sample.get("__key__", "unknown") if isinstance(sample, dict) else "unknown"
                logger.warning(f"Low quality image {key} is skipped in Flux Dataloader.")
                continue
            p = self.classifier_free_guidance_prob
            if p > 0.0:
                if float(torch.rand(1, generator=self._gen)) < p:
                    out["t5_tokens"] = self._t5_empty
                if float(torch.rand(1, generator=self._gen)) < p:
                    out["clip_tokens"] = self._clip_empty
            for k in ("t5_tokens", "clip_tokens"):             # one row per sample: [1, L] -> [L]
                if torch.is_tensor(out[k]) and out[k].dim() == 2 and out[k].shape[0] == 1:
                    out[k] = out[k][0]
            labels = out.pop("image")
            yield out, labels

    def state_dict(self):
        state = {"rng": self._gen.get_state()}
        if self._own_state():
            state["data"] = self._data.state_dict()
        else:
            state["sample_idx"] = self._sample_idx
        return state

    def load_state_dict(self, state_dict):
        self._restored = True
        if "rng" in state_dict:
            self._gen.set_state(state_dict["rng"])
        if self._own_state():
            assert "data" in state_dict
            self._data.load_state_dict(state_dict["data"])
        else:
            self._sample_idx = int(state_dict.get("sample_idx", state_dict.get("consumed", 0)))


class FluxValidationDataset(FluxDataset):
    """Adds to every sample one of eight stratified noise levels ``(i + 0.5) / 8`` in turn, the validation protocol of
    the SD3 paper (torchtitan/models/flux/flux_datasets.py:330-384)."""

    def __init__(self, *args, generate_timesteps: bool = True, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        self.generate_timesteps = generate_timesteps
        self._levels = itertools.cycle([(i + 0.5) / 8 for i in range(8)])

    def __iter__(self):
        for inputs, labels in super().__iter__():
            if self.generate_timesteps:
                inputs["timestep"] = next(self._levels)
            yield inputs, labels


class SyntheticFluxDataset(IterableDataset):
    """Random images and token ids, a different stream per data-parallel rank; both token rows are zeroed together with
    probability ``cfg_prob``; ``generate_timesteps`` attaches the stratified validation noise levels in turn. A loader
    that is not ``infinite`` gets 256 samples per rank."""

    def __init__(self, img_size: int, t5_len: int, clip_len: int, cfg_prob: float, rank: int, world: int, seed: int = 0,
                 t5_vocab: int = 32128, clip_vocab: int = 49408, generate_timesteps: bool = False, length: int | None = None):
        self.length = length                                   # samples per rank before the stream ends; None = endless
        self.img_size, self.t5_len, self.clip_len, self.cfg_prob = img_size, t5_len, clip_len, cfg_prob
        self.rank, self.world, self.seed, self.t5_vocab, self.clip_vocab = rank, world, seed, t5_vocab, clip_vocab
        self.generate_timesteps = generate_timesteps
        self._n = 0

    def _sample(self, n: int):
        g = torch.Generator().manual_seed((self.seed * 7919 + self.rank) * 1_000_003 + n)
        h = int(torch.randint(self.img_size, 2 * self.img_size, (1,), generator=g))
        w = int(torch.randint(self.img_size, 2 * self.img_size, (1,), generator=g))
        img = process_image(torch.rand(3, h, w, generator=g), self.img_size)
        empty = bool(torch.rand((), generator=g) < self.cfg_prob)
        t5 = torch.zeros(self.t5_len, dtype=torch.long) if empty else torch.randint(1, self.t5_vocab, (self.t5_len,), generator=g)
        clip = torch.zeros(self.clip_len, dtype=torch.long) if empty else torch.randint(1, self.clip_vocab, (self.clip_len,), generator=g)
        inputs = {"clip_tokens": clip, "t5_tokens": t5}
        if self.generate_timesteps:
            inputs["timestep"] = (n % 8 + 0.5) / 8
        return inputs, img

    def __iter__(self):
        # sample n depends on (seed, rank, n) only: a restored loader continues exactly, loader workers take every k-th
        wid, workers = _worker()
        while self.length is None or self._n < self.length:
            n = self._n
            self._n += 1
            if n % workers == wid:
                yield self._sample(n)

    def state_dict(self):
        return {"n": self._n}

    def load_state_dict(self, sd):
        self._n = sd.get("n", 0)


# ------------------------------------------------------------------------------------------ loader
def _collate(items):
    first = items[0][0]
    inputs = {}
    for k in first:
        vals = [i[0][k] for i in items]
        if torch.is_tensor(vals[0]):
            inputs[k] = torch.stack(vals)
        elif isinstance(vals[0], float):
            inputs[k] = torch.tensor(vals)
        else:
            inputs[k] = vals
    return inputs, torch.stack([i[1] for i in items])


class FluxDataLoader(ParallelAwareDataloader):
    """The FLUX dataset behind the stateful, worker-capable loader of the text pipeline: ``--dataloader.num_workers``
    moves image decoding and resizing into worker processes; the loader state (per data-parallel rank) is part of the
    checkpoint (torchtitan/models/flux/flux_datasets.py:387-463)."""

    @dataclass(kw_only=True, slots=True)
    class Config(ParallelAwareDataloader.Config):
        dataset: str = "cc12m-test"
        """``synthetic`` or a name registered in ``DATASETS``."""
        dataset_path: str | None = None
        """Local copy (or another hub name); default: the registry entry's path."""
        classifier_free_guidance_prob: float = 0.1
        """Each text encoding is dropped independently with this probability: with two encoders and p = 0.447 the
        unconditional model is trained in 20 % of the steps."""
        img_size: int = 256
        generate_timesteps: bool = False
        """Attach stratified noise levels in turn (validation)."""
        t5_max_length: int = 256
        clip_max_length: int = 77
        t5_tokenizer_path: str | None = None
        clip_tokenizer_path: str | None = None
        test_tokenizer: bool = False
        """Use the asset-free tokenizer (also chosen when the tokenizer folders are missing)."""
        encoder: Encoder = field(default_factory=Encoder)
        """The reference's way to name the tokenizer folders (``--dataloader.encoder.t5_encoder`` ...); used where the
        fields above are not set."""
        hf_assets_path: str = "./tests/assets/tokenizer"
        """Accepted for command lines written for the reference, which reads its test tokenizer from here; the asset-free
        tokenizer of this framework needs no files."""
        infinite: bool = True
        seed: int = 0

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, local_batch_size: int, **kwargs):
        self.config = config
        if config.dataset == "synthetic":
            ds = SyntheticFluxDataset(config.img_size, config.t5_max_length, config.clip_max_length,
                                                config.classifier_free_guidance_prob, dp_rank, dp_world_size, seed=config.seed,
                                                generate_timesteps=config.generate_timesteps,
                                                length=None if config.infinite else 256)
        else:
            from .tokenizer import build_flux_tokenizer

            enc = config.encoder
            t5, clip = build_flux_tokenizer(
                t5_path=config.t5_tokenizer_path or enc.t5_encoder, clip_path=config.clip_tokenizer_path or enc.clip_encoder,
                t5_max_length=enc.max_t5_encoding_len if config.t5_max_length == 256 else config.t5_max_length,
                clip_max_length=config.clip_max_length, test_mode=config.test_tokenizer or enc.test_mode)
            cls = FluxValidationDataset if config.generate_timesteps else FluxDataset
            ds = cls(config.dataset, config.dataset_path, t5, clip, config.classifier_free_guidance_prob,
                               config.img_size, dp_rank, dp_world_size, infinite=config.infinite, seed=config.seed)
        super().__init__(ds, dp_rank=dp_rank, dp_world_size=dp_world_size, batch_size=local_batch_size, collate_fn=_collate,
                         num_workers=config.num_workers, persistent_workers=config.persistent_workers,
                         pin_memory=config.pin_memory, prefetch_factor=config.prefetch_factor)
