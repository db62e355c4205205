"""Image-text datasets for the vision-language trainer: OBELICS-style interleaved documents and CC12M-style
image-caption pairs read through the ``datasets`` library (streaming or local files), decoded, resized to a
patch-multiple at native aspect ratio, tokenised, packed and checkpointed.

What it reproduces from torchtitan/experiments/vlm/datasets/mm_datasets.py:36-330 and datasets/utils/{image,text,
packing}.py: a registry of named datasets (``obelics``, ``cc12m``, ``cc12m-test``) each with a loader and a sample
adapter; every sample becomes ``texts`` / ``images`` lists of equal length in which ``None`` marks the other modality's
position (a caption pair is the interleaved document ``[image, text]``); an image becomes ``<boi> <img> * L <eoi>`` in
the token stream with ``L`` its patch count after spatial merging; labels ignore the three image tokens and padding;
samples longer than the sequence are dropped with a warning; a sample whose images cannot all be decoded is dropped;
the stream is split over data-parallel ranks with ``split_dataset_by_node``; the loader state is the number of samples
consumed plus the packer's content.

Different from the reference: packing is first-fit-decreasing over a buffer of ``packing_buffer_size`` samples (the
buffer is emptied whenever it fills), and one packed row carries its images with it, so the collator of
``datasets.py`` is shared with the synthetic stream.
"""

from __future__ import annotations

import io
from dataclasses import dataclass
from typing import Any, Callable

import torch

from torchtitan_b200.tools.logging import logger

from .datasets import patchify, smart_resize
from .model import SpecialTokens

__all__ = ["MM_DATASETS", "MMDatasetSpec", "register_mm_dataset", "decode_image", "process_document", "BufferedPacker",
           "InterleavedDataset"]

# SigLIP-2 preprocessing: pixels scaled to [-1, 1]
_MEAN, _STD = 0.5, 0.5


def decode_image(raw) -> torch.Tensor | None:
    """bytes / ``{"bytes": ...}`` / PIL image / [C, H, W] tensor -> float tensor [3, H, W] in [0, 1]; None when it cannot
    be decoded."""
    if raw is None:
        return None
    if torch.is_tensor(raw):
        return raw.float()
    try:
        from PIL import Image

        if isinstance(raw, dict):
            raw = raw.get("bytes") or raw.get("path")
        if isinstance(raw, (bytes, bytearray)):
            raw = Image.open(io.BytesIO(raw))
        elif isinstance(raw, str):
            raw = Image.open(raw)
        img = raw.convert("RGB")
        data = torch.frombuffer(bytearray(img.tobytes()), dtype=torch.uint8).view(img.height, img.width, 3)
        return data.permute(2, 0, 1).float() / 255.0
    except Exception as e:  # a broken download is a data problem, not a crash
        logger.warning(f"cannot decode image: {e}")
        return None


def process_document(texts, images, tokenizer, st: SpecialTokens, *, patch: int, max_patches: int, merge: int = 1):
    """One interleaved document -> (token ids, [patches [L, 3 * patch^2]], [grids [L, 3]]) or None when it has to be
    dropped. ``texts[i]`` is None where ``images[i]`` holds an image and the other way round."""
    if isinstance(texts, str):
        texts = [texts]
    if not isinstance(images, (list, tuple)):
        images = [images]
    if not texts or len(texts) != len(images):
        return None
    ids: list[int] = []
    pats, grids = [], []
    for text, raw in zip(texts, images):
        if raw is not None:
            img = decode_image(raw)
            if img is None or img.dim() != 3 or min(img.shape[1:]) < 1:
                logger.warning("cannot process every image of a sample: dropped")
                return None
            H, W = smart_resize(img.shape[1], img.shape[2], patch, max_patches, merge)
            img = torch.nn.functional.interpolate(img.unsqueeze(0), size=(H, W), mode="bilinear", align_corners=False,
                                                  antialias=True)[0]
            p, g = patchify((img - _MEAN) / _STD, patch)
            pats.append(p)
            grids.append(g)
            ids += [st.boi_id] + [st.img_id] * (p.shape[0] // (merge * merge)) + [st.eoi_id]
        elif text:
            ids += tokenizer.encode(text, add_bos=False, add_eos=False)
    if not ids:
        return None
    eos = getattr(tokenizer, "eos_id", None)
    if eos is not None:
        ids.append(eos)
    return ids, pats, grids


class BufferedPacker:
    """Packs whole samples into rows of ``seq_len + 1`` tokens. Samples collect in a buffer of ``buffer_size``; when it
    is full they are placed first-fit in order of decreasing length and every row comes out. ``buffer_size = 0`` turns
    packing off: one sample per row. Rows are ``(ids padded to seq_len + 1, [patches], [grids])``."""

    def __init__(self, seq_len: int, st: SpecialTokens, buffer_size: int):
        self.row_len, self.st, self.buffer_size = seq_len + 1, st, buffer_size
        self.buffer: list = []
        self.ready: list = []

    def _row(self, ids, pats, grids):
        return (list(ids) + [self.st.pad_id] * (self.row_len - len(ids)), list(pats), list(grids))

    def add(self, sample) -> None:
        if self.buffer_size <= 0:
            self.ready.append(self._row(*sample))
            return
        self.buffer.append(sample)
        if len(self.buffer) >= self.buffer_size:
            self.flush()

    def flush(self) -> None:
        bins: list = []
        for ids, pats, grids in sorted(self.buffer, key=lambda s: -len(s[0])):
            for b in bins:
                if len(b[0]) + len(ids) <= self.row_len:
                    b[0].extend(ids); b[1].extend(pats); b[2].extend(grids)
                    break
            else:
                bins.append([list(ids), list(pats), list(grids)])
        self.ready.extend(self._row(*b) for b in bins)
        self.buffer = []

    def pop(self):
        return self.ready.pop(0) if self.ready else None

    def state_dict(self):
        return {"buffer": list(self.buffer), "ready": list(self.ready)}

    def load_state_dict(self, state):
        self.buffer, self.ready = list(state.get("buffer", [])), list(state.get("ready", []))


# ------------------------------------------------------------------------------------------ registry
@dataclass
class MMDatasetSpec:
    path: str
    loader: Callable[[str], Any]                       # path -> an (iterable) dataset of raw samples
    adapter: Callable[[dict], tuple[list, list]]       # raw sample -> (texts, images) of equal length


def _load_stream(path: str):
    from datasets import load_dataset

    return load_dataset(path, split="train", streaming=True)


def _load_tar_folder(path: str):
    """A folder of WebDataset shards (``*.tar`` holding ``<key>.jpg`` / ``<key>.txt`` pairs)."""
    from datasets import load_dataset

    return load_dataset("webdataset", data_files={"train": f"{path}/*.tar"}, split="train", streaming=True)


def _interleaved(sample: dict):
    return sample.get("texts", []), sample.get("images", [])


def _caption_pair(sample: dict):
    # an image followed by its caption is an interleaved document of two entries
    return [None, sample.get("txt", "")], [sample.get("jpg"), None]


MM_DATASETS: dict[str, MMDatasetSpec] = {
    "obelics": MMDatasetSpec("HuggingFaceM4/OBELICS", _load_stream, _interleaved),
    "cc12m": MMDatasetSpec("pixparse/cc12m-wds", _load_stream, _caption_pair),
    "cc12m-test": MMDatasetSpec("tests/assets/cc12m_test", _load_tar_folder, _caption_pair),
}


def register_mm_dataset(name: str, spec: MMDatasetSpec) -> None:
    MM_DATASETS[name.lower()] = spec


class InterleavedDataset(torch.utils.data.IterableDataset):
    """Rows for the collator from a named image-text dataset, this data-parallel rank's share of it."""

    def __init__(self, name: str, path: str | None, tokenizer, st: SpecialTokens, *, seq_len: int, patch: int,
                 max_patches: int, merge: int = 1, packing_buffer_size: int = 0, dp_rank: int = 0, dp_world_size: int = 1,
                 infinite: bool = False):
        name = name.lower()
        if name not in MM_DATASETS:
            raise ValueError(f"Dataset {name} is not supported. Supported datasets are: {list(MM_DATASETS.keys())}")
        spec = MM_DATASETS[name]
        path = path or spec.path
        logger.info(f"Preparing {name} dataset from {path}")
        data = spec.loader(path)
        if dp_world_size > 1:
            from datasets.distributed import split_dataset_by_node

            data = split_dataset_by_node(data, dp_rank, dp_world_size)
        self._data, self._adapter = data, spec.adapter
        self.tokenizer, self.st, self.seq_len = tokenizer, st, seq_len
        self.patch, self.max_patches, self.merge, self.infinite = patch, max_patches, merge, infinite
        self.packer = BufferedPacker(seq_len, st, packing_buffer_size)
        self._sample_idx = 0

    def _raw_samples(self):
        it = iter(self._data)
        for _ in range(self._sample_idx):          # resume: skip what earlier steps consumed
            if next(it, None) is None:
                return
        yield from it

    def __iter__(self):
        while True:
            row = self.packer.pop()                 # rows restored from a checkpoint come first
            while row is not None:
                yield row
                row = self.packer.pop()
            for raw in self._raw_samples():
                self._sample_idx += 1
                try:
                    texts, images = self._adapter(raw)
                    doc = process_document(texts, images, self.tokenizer, self.st, patch=self.patch,
                                           max_patches=self.max_patches, merge=self.merge)
                except Exception as e:
                    logger.warning(f"Error processing sample: {e}")
                    continue
                if doc is None:
                    continue
                if len(doc[0]) > self.seq_len:
                    logger.warning(f"Sample length {len(doc[0])} > training seq_len={self.seq_len}. Skip")
                    continue
                self.packer.add(doc)
                row = self.packer.pop()
                while row is not None:
                    yield row
                    row = self.packer.pop()
            self.packer.flush()
            row = self.packer.pop()
            while row is not None:
                yield row
                row = self.packer.pop()
            if not self.infinite:
                return
            self._sample_idx = 0

    def state_dict(self):
        return {"sample_idx": self._sample_idx, "packer": self.packer.state_dict()}

    def load_state_dict(self, state):
        self._sample_idx = int(state.get("sample_idx", 0))
        self.packer.load_state_dict(state.get("packer", {}))
