"""Prompt tokenizers for FLUX: a T5 and a CLIP tokenizer, each padding / truncating to a fixed length and returning int64
ids ``[1, max_length]``. ``FluxTokenizer`` wraps a Hugging Face tokenizer loaded from a local folder; ``FluxTestTokenizer``
needs no assets (stable hash of whitespace-separated words), which is what the offline configs and the tests use.
Parity: torchtitan/models/flux/tokenizer.py (FluxTokenizer, FluxTestTokenizer, build_flux_tokenizer)."""

from __future__ import annotations

import hashlib
import os

import torch

from torchtitan_b200.tools.logging import logger

from torchtitan_b200.components.tokenizer import BaseTokenizer


class FluxTestTokenizer(BaseTokenizer):
    """Asset-free tokenizer: word -> 1 + (md5(word) mod (vocab - 2)); 0 pads, ``vocab - 1`` ends the prompt."""

    def __init__(self, max_length: int = 77, vocab_size: int = 32128, **kwargs):
        super().__init__()
        self._max_length, self._vocab = max_length, vocab_size
        self.pad_id, self.eos_id = 0, vocab_size - 1

    def _word(self, w: str) -> int:
        return 1 + int.from_bytes(hashlib.md5(w.encode()).digest()[:8], "little") % (self._vocab - 2)

    def encode(self, text: str | list[str], **kwargs) -> torch.Tensor:
        texts = [text] if isinstance(text, str) else list(text)
        out = torch.full((len(texts), self._max_length), self.pad_id, dtype=torch.long)
        for i, t in enumerate(texts):
            ids = [self._word(w) for w in t.split()][: self._max_length - 1] + [self.eos_id]
            out[i, : len(ids)] = torch.tensor(ids, dtype=torch.long)
        return out

    def decode(self, token_ids, **kwargs) -> str:
        ids = token_ids.flatten().tolist() if torch.is_tensor(token_ids) else list(token_ids)
        return " ".join(f"<{i}>" for i in ids if i not in (self.pad_id, self.eos_id))

    def get_vocab_size(self) -> int:
        return self._vocab


class FluxTokenizer(BaseTokenizer):
    """A Hugging Face CLIP or T5 tokenizer from a local folder (``transformers`` is imported only here)."""

    def __init__(self, model_path: str, max_length: int = 77, **hf_kwargs):
        super().__init__()
        if not os.path.isdir(model_path):
            raise FileNotFoundError(f"tokenizer folder {model_path} not found (download it with scripts/download_hf_assets.py)")
        from transformers import AutoTokenizer

        self._tok = AutoTokenizer.from_pretrained(model_path, local_files_only=True, **hf_kwargs)
        self._max_length = max_length

    def encode(self, text: str | list[str], **kwargs) -> torch.Tensor:
        enc = self._tok(text, truncation=True, max_length=self._max_length, return_length=False,
                        return_overflowing_tokens=False, padding="max_length", return_tensors="pt")
        return enc["input_ids"].long()

    def decode(self, token_ids, **kwargs) -> str:
        return self._tok.decode(token_ids.flatten().tolist() if torch.is_tensor(token_ids) else token_ids, skip_special_tokens=True)

    def get_vocab_size(self) -> int:
        return len(self._tok)


def build_flux_tokenizer(*, t5_path: str | None, clip_path: str | None, t5_max_length: int = 256, clip_max_length: int = 77,
                         test_mode: bool = False):
    """(t5 tokenizer, clip tokenizer); ``test_mode`` or missing folders select the asset-free tokenizer."""
    def one(path, length, vocab):
        if test_mode or path is None or not os.path.isdir(path):
            if not test_mode and path is not None:
                logger.warning(f"tokenizer folder {path!r} not found: using the asset-free test tokenizer")
            return FluxTestTokenizer(max_length=length, vocab_size=vocab)
        return FluxTokenizer(path, max_length=length)

    return one(t5_path, t5_max_length, 32128), one(clip_path, clip_max_length, 49408)
