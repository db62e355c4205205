"""Multimodal data path: native-resolution patchification, sample packing, collation
(torchtitan/experiments/vlm/datasets/{mm_datasets,mm_collator_nld}.py and datasets/utils/{image,packing,text}.py)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from torchtitan_b200.components.dataloader import ParallelAwareDataloader

from .model import SpecialTokens


def smart_resize(h: int, w: int, patch: int, max_patches: int, merge: int = 1) -> tuple[int, int]:
    """Closest size that is a multiple of ``patch * merge`` per side, keeps the aspect ratio and has <= ``max_patches`` patches."""
    unit = patch * merge
    H, W = max(unit, round(h / unit) * unit), max(unit, round(w / unit) * unit)
    if (H // patch) * (W // patch) > max_patches:
        scale = (max_patches * patch * patch / (h * w)) ** 0.5
        H, W = max(unit, int(h * scale) // unit * unit), max(unit, int(w * scale) // unit * unit)
    return H, W


def patchify(img_chw: torch.Tensor, patch: int) -> tuple[torch.Tensor, torch.Tensor]:
    """[C, H, W] -> (patches [L, C*patch*patch], grid [L, 3] of (t, h, w) coordinates)."""
    C, H, W = img_chw.shape
    gh, gw = H // patch, W // patch
    p = img_chw.reshape(C, gh, patch, gw, patch).permute(1, 3, 0, 2, 4).reshape(gh * gw, C * patch * patch)
    hh, ww = torch.meshgrid(torch.arange(gh), torch.arange(gw), indexing="ij")
    grid = torch.stack((torch.zeros_like(hh), hh, ww), dim=-1).reshape(-1, 3)
    return p, grid


def process_sample(text_ids_before: list[int], images: list[torch.Tensor], text_ids_after: list[int], st: SpecialTokens,
                   patch: int, max_patches: int):
    """One document: ``<text> (<boi> <image>*L <eoi>)* <text>``; returns (token ids, [patches], [grids])."""
    ids, pats, grids = list(text_ids_before), [], []
    for img in images:
        H, W = smart_resize(img.shape[1], img.shape[2], patch, max_patches)
        img = torch.nn.functional.interpolate(img.unsqueeze(0).float(), size=(H, W), mode="bilinear", align_corners=False)[0]
        p, g = patchify(img, patch)
        pats.append(p)
        grids.append(g)
        ids += [st.boi_id] + [st.img_id] * p.shape[0] + [st.eoi_id]
    return ids + list(text_ids_after), pats, grids


class SamplePacker:
    """Greedy packing of whole samples into sequences of ``seq_len + 1`` tokens (a sample that does not fit starts the
    next sequence; over-long samples are truncated and lose their images past the cut)."""

    def __init__(self, seq_len: int, st: SpecialTokens):
        self.seq_len, self.st = seq_len + 1, st
        self.ids: list[int] = []
        self.pats: list[torch.Tensor] = []
        self.grids: list[torch.Tensor] = []

    def add(self, ids, pats, grids):
        out = None
        if len(self.ids) + len(ids) > self.seq_len and self.ids:
            out = self.flush()
        if len(ids) > self.seq_len:
            ids = ids[: self.seq_len]
            kept = sum(1 for t in ids if t == self.st.img_id)
            n, keep_p, keep_g = 0, [], []
            for p, g in zip(pats, grids):
                if n + p.shape[0] <= kept:
                    keep_p.append(p)
                    keep_g.append(g)
                    n += p.shape[0]
            ids = [t if (t != self.st.img_id or i < 0) else t for i, t in enumerate(ids)]
            # placeholders without a complete image become padding
            extra = kept - n
            if extra:
                idx = [i for i, t in enumerate(ids) if t == self.st.img_id][-extra:]
                for i in idx:
                    ids[i] = self.st.pad_id
            pats, grids = keep_p, keep_g
        self.ids += ids
        self.pats += pats
        self.grids += grids
        return out

    def flush(self):
        ids = self.ids + [self.st.pad_id] * (self.seq_len - len(self.ids))
        out = (ids, self.pats, self.grids)
        self.ids, self.pats, self.grids = [], [], []
        return out


@dataclass
class MultiModalCollatorNLD:
    """Stack packed sequences; images of the whole batch form ``pixel_values [N, L, D]`` / ``grid_thw [N, L, 3]`` padded
    with -1 coordinates, N padded to ``max_images_per_batch`` so that shapes are static."""

    patch_dim: int
    max_images_per_batch: int
    max_patches_per_image: int
    special_tokens: SpecialTokens

    def __call__(self, batch):
        st = self.special_tokens
        toks = torch.tensor([b[0] for b in batch], dtype=torch.long)
        N, L = self.max_images_per_batch, self.max_patches_per_image
        pixels = torch.zeros(N, L, self.patch_dim)
        grid = torch.full((N, L, 3), -1, dtype=torch.long)
        n = 0
        for _, pats, grids in batch:
            for p, g in zip(pats, grids):
                assert n < N, "more images in the batch than max_images_per_batch"
                pixels[n, : p.shape[0]] = p
                grid[n, : g.shape[0]] = g
                n += 1
        inputs, labels = toks[:, :-1], toks[:, 1:].clone()
        # the shift drops the last token of every row; where that token was an image placeholder, drop the patch it stood
        # for as well (the last patch of the row's last image), so placeholders and patches stay one to one
        n = 0
        for b, (_, pats, _) in enumerate(batch):
            n += len(pats)
            if len(pats) and int(toks[b, -1]) == st.img_id:
                valid = (grid[n - 1, :, 1:] != -1).all(-1).nonzero()
                if valid.numel():
                    grid[n - 1, int(valid[-1])] = -1
        for t in (st.pad_id, st.img_id, st.boi_id, st.eoi_id):
            labels[labels == t] = st.ignore_id
        return {"input": inputs, "pixel_values": pixels, "grid_thw": grid, "special_tokens": st}, labels


class SyntheticMultiModalDataset(torch.utils.data.IterableDataset):
    """Random text and random images of varying aspect ratio (offline stand-in for OBELICS / CC12M streams). The stream
    is a pure function of (seed, rank, loader worker); its state is the number of rows handed out, and a restored copy
    regenerates and skips that many."""

    def __init__(self, st: SpecialTokens, vocab: int, seq_len: int, patch: int = 16, max_patches: int = 64, seed: int = 0,
                 dp_rank: int = 0, dp_world_size: int = 1):
        self.st, self.vocab, self.seq_len, self.patch, self.max_patches = st, vocab, seq_len, patch, max_patches
        self.seed, self.rank, self.world = seed, dp_rank, dp_world_size
        self._rows = 0

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        wid = info.id if info is not None else 0
        g = torch.Generator().manual_seed((self.seed * 1000 + self.rank) * 64 + wid)
        packer = SamplePacker(self.seq_len, self.st)
        reserved = {self.st.img_id, self.st.boi_id, self.st.eoi_id, self.st.pad_id}
        skip, self._rows = self._rows, 0
        while True:
            n_txt = int(torch.randint(8, 64, (1,), generator=g))
            ids = [t for t in torch.randint(0, self.vocab, (n_txt,), generator=g).tolist() if t not in reserved]
            imgs = []
            for _ in range(int(torch.randint(0, 3, (1,), generator=g))):
                h = int(torch.randint(2, 8, (1,), generator=g)) * self.patch
                w = int(torch.randint(2, 8, (1,), generator=g)) * self.patch
                imgs.append(torch.rand(3, h, w, generator=g))
            sample = process_sample(ids[: n_txt // 2], imgs, ids[n_txt // 2 :], self.st, self.patch, self.max_patches)
            out = packer.add(*sample)
            if out is not None:
                self._rows += 1
                if self._rows > skip:
                    yield out

    def state_dict(self):
        return {"rows": self._rows}

    def load_state_dict(self, state):
        self._rows = int(state.get("rows", 0))


class MMDataLoader(ParallelAwareDataloader):
    """Packed multimodal batches for the trainer: ``({"input", "pixel_values", "grid_thw", "special_tokens"}, labels)``.

    Reference: torchtitan/experiments/vlm/datasets/mm_datasets.py:370-453 (the loader built from the job configuration,
    on the stateful loader of the text pipeline: ``num_workers`` moves image decoding into worker processes and the
    loader state per data-parallel rank goes into the checkpoint). The ``synthetic`` dataset needs no files; when the
    tokenizer has no image tokens the special tokens take the last four ids of the model's vocabulary."""

    @dataclass(kw_only=True, slots=True)
    class Config(ParallelAwareDataloader.Config):
        dataset: str = "cc12m-test"
        """``synthetic``, or a name registered in ``mm_datasets.MM_DATASETS`` (``obelics``, ``cc12m``, ``cc12m-test``)."""
        dataset_path: str | None = None
        infinite: bool = True
        max_images_per_batch: int = 10
        """Vision encoder batch: images beyond it are dropped from the batch with a warning."""
        max_patches_per_image: int = 256
        """Larger images are scaled down keeping the aspect ratio."""
        patch_size: int = 16
        spatial_merge_size: int = 1
        packing_buffer_size: int = 0
        """Samples buffered for packing several into one row; 0 = one sample per row."""
        seed: int = 0

    def __init__(self, config: Config, *, dp_world_size: int, dp_rank: int, tokenizer=None, seq_len: int, local_batch_size: int,
                 model_vocab_size: int | None = None, **kwargs):
        self.config = config
        try:
            st = SpecialTokens.from_tokenizer(tokenizer)
        except Exception:
            v = model_vocab_size or 2048
            st = SpecialTokens("<|image|>", v - 4, "<|begin_of_image|>", v - 3, "<|end_of_image|>", v - 2, "<|pad|>", v - 1)
        self.special_tokens = st
        self.synthetic = config.dataset == "synthetic"
        if self.synthetic:
            vocab = min(i for i in (st.img_id, st.boi_id, st.eoi_id, st.pad_id))
            ds = SyntheticMultiModalDataset(st, vocab=vocab, seq_len=seq_len, patch=config.patch_size,
                                            max_patches=config.max_patches_per_image, seed=config.seed,
                                            dp_rank=dp_rank, dp_world_size=dp_world_size)
        else:
            from .mm_datasets import InterleavedDataset

            assert tokenizer is not None, "image-text datasets need a tokenizer"
            if config.spatial_merge_size != 1:
                raise NotImplementedError("spatial_merge_size > 1: the projector of this model does not merge patches")
            ds = InterleavedDataset(config.dataset, config.dataset_path, tokenizer, st, seq_len=seq_len,
                                    patch=config.patch_size, max_patches=config.max_patches_per_image,
                                    merge=config.spatial_merge_size, packing_buffer_size=config.packing_buffer_size,
                                    dp_rank=dp_rank, dp_world_size=dp_world_size, infinite=config.infinite)
        self.collate = MultiModalCollatorNLD(patch_dim=3 * config.patch_size ** 2, max_images_per_batch=config.max_images_per_batch,
                                             max_patches_per_image=config.max_patches_per_image, special_tokens=st)
        # a finite dataset's last short batch is dropped: the collator pads to fixed image counts, not to a batch size
        super().__init__(ds, dp_rank=dp_rank, dp_world_size=dp_world_size, batch_size=local_batch_size, collate_fn=self.collate,
                         drop_last=True, num_workers=config.num_workers, persistent_workers=config.persistent_workers,
                         pin_memory=config.pin_memory, prefetch_factor=config.prefetch_factor)


#: the reference's name for the loader class
HuggingFaceMultiModalDataLoader = MMDataLoader
