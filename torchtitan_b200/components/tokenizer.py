"""Tokenizers.

Parity: torchtitan/components/tokenizer.py:19-503. ``BaseTokenizer`` defines encode/decode/
vocab size plus sandboxed Jinja chat templates; ``HuggingFaceTokenizer`` loads ``tokenizer.json``
(or ``vocab.json``/``vocab.txt`` with optional ``merges.txt``) from a local folder, reads BOS/EOS
from ``tokenizer_config.json`` / ``config.json`` / ``generation_config.json``, and probes the
underlying tokenizer once to learn whether it already inserts BOS/EOS so that
``encode(add_bos=..., add_eos=...)`` never doubles them.
"""

from __future__ import annotations

import json
import os
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any

from torchtitan_b200.config.configurable import Configurable
from torchtitan_b200.tools.logging import logger


class BaseTokenizer(ABC, Configurable):
    @dataclass(kw_only=True, slots=True)
    class Config(Configurable.Config):
        pass

    def __init__(self):
        self.eos_id = 0
        self.chat_template: str | None = None
        self._jinja_template = None

    @abstractmethod
    def encode(self, *args, **kwargs) -> list[int]: ...

    @abstractmethod
    def decode(self, *args, **kwargs) -> str: ...

    @abstractmethod
    def get_vocab_size(self) -> int: ...

    def set_chat_template(self, template: str) -> None:
        import datetime

        from jinja2.exceptions import TemplateError
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(msg):
            raise TemplateError(msg)

        def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
            return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.filters["tojson"] = tojson
        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        self.chat_template = template
        self._jinja_template = env.from_string(template)

    def apply_chat_template(self, messages: list[dict[str, str]], **kwargs) -> str:
        if self._jinja_template is None:
            raise ValueError("No chat template set. Call set_chat_template() first or provide chat_template in tokenizer_config.json")
        ctx = dict(messages=messages, add_generation_prompt=kwargs.pop("add_generation_prompt", False),
                   bos_token=getattr(self, "bos_token", None) or "", eos_token=getattr(self, "eos_token", None) or "")
        ctx.update(kwargs)
        return self._jinja_template.render(**ctx)


class HuggingFaceTokenizer(BaseTokenizer):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseTokenizer.Config):
        pass

    def __init__(self, config: Config | None = None, *, tokenizer_path: str, **kwargs):
        super().__init__()
        self.tokenizer_path = tokenizer_path
        self.tokenizer = self._load_tokenizer_from_path(tokenizer_path)
        self.config = self._load_json(os.path.join(tokenizer_path, "tokenizer_config.json"))
        self.bos_id = self.eos_id = None
        self.bos_token = self.eos_token = None
        self._infer_special_tokens()
        self._infer_should_add_bos_eos()
        if self.config and self.config.get("chat_template"):
            self.set_chat_template(self.config["chat_template"])

    @staticmethod
    def _load_json(path: str) -> dict | None:
        if os.path.exists(path):
            with open(path) as f:
                return json.load(f)
        return None

    def _load_tokenizer_from_path(self, path: str):
        from tokenizers import Tokenizer

        if not os.path.exists(path):
            raise FileNotFoundError(f"Tokenizer path '{path}' does not exist")
        if os.path.isfile(path):
            return Tokenizer.from_file(path)
        tj = os.path.join(path, "tokenizer.json")
        if os.path.exists(tj):
            logger.info("Loading tokenizer from tokenizer.json")
            return Tokenizer.from_file(tj)
        vocab_json, vocab_txt = os.path.join(path, "vocab.json"), os.path.join(path, "vocab.txt")
        merges = os.path.join(path, "merges.txt")
        if os.path.exists(vocab_json) or os.path.exists(vocab_txt):
            from tokenizers.models import BPE, WordLevel

            if os.path.exists(vocab_json):
                with open(vocab_json) as f:
                    vocab = json.load(f)
            else:
                with open(vocab_txt) as f:
                    vocab = {line.split("\t" if "\t" in line else " ")[0].strip(): i for i, line in enumerate(f) if line.strip()}
            if os.path.exists(merges):
                pairs = []
                with open(merges) as f:
                    for line in f:
                        line = line.strip()
                        if line and not line.startswith("#"):
                            a, b = line.split(" ", 1)
                            pairs.append((a, b))
                logger.info("Loading tokenizer from vocab + merges")
                return Tokenizer(BPE(vocab=vocab, merges=pairs))
            logger.info("Loading tokenizer from vocab only")
            return Tokenizer(WordLevel(vocab=vocab, unk_token="[UNK]"))
        raise FileNotFoundError(
            f"No supported tokenizer files found in '{path}'. Available files: {sorted(os.listdir(path))}. "
            "Looking for: tokenizer.json, vocab.json/vocab.txt (+ merges.txt)"
        )

    @staticmethod
    def _token_str(cfg: dict | None, key: str) -> str | None:
        if not cfg:
            return None
        v = cfg.get(key)
        if isinstance(v, dict):
            return v.get("content")
        return v if isinstance(v, str) else None

    def _infer_special_tokens(self):
        self.bos_token = self._token_str(self.config, "bos_token")
        self.eos_token = self._token_str(self.config, "eos_token")
        added = {}
        if self.config and isinstance(self.config.get("added_tokens_decoder"), dict):
            added = {v.get("content"): int(k) for k, v in self.config["added_tokens_decoder"].items()}
        def lookup(tok):
            if tok is None:
                return None
            tid = self.tokenizer.token_to_id(tok)
            return tid if tid is not None else added.get(tok)
        self.bos_id, self.eos_id = lookup(self.bos_token), lookup(self.eos_token)
        # fall back to ids in config.json / generation_config.json
        for fname in ("config.json", "generation_config.json"):
            cfg = self._load_json(os.path.join(self.tokenizer_path, fname)) if os.path.isdir(self.tokenizer_path) else None
            if not cfg:
                continue
            if self.bos_id is None and isinstance(cfg.get("bos_token_id"), int):
                self.bos_id = cfg["bos_token_id"]
            if self.eos_id is None:
                e = cfg.get("eos_token_id")
                self.eos_id = e if isinstance(e, int) else (e[0] if isinstance(e, list) and e else None)
        if self.bos_token is None and self.bos_id is not None:
            self.bos_token = self.tokenizer.id_to_token(self.bos_id)
        if self.eos_token is None and self.eos_id is not None:
            self.eos_token = self.tokenizer.id_to_token(self.eos_id)

    def _infer_should_add_bos_eos(self):
        """Encode an empty string with the tokenizer's own post-processing to see what it adds."""
        self.default_add_bos = self.default_add_eos = False
        self.hf_adds_bos = self.hf_adds_eos = False
        probe = self.tokenizer.encode("", add_special_tokens=True).ids
        if self.bos_id is not None and self.bos_id in probe:
            self.hf_adds_bos = True
        if self.eos_id is not None and self.eos_id in probe:
            self.hf_adds_eos = True
        if self.config:
            self.default_add_bos = bool(self.config.get("add_bos_token", self.hf_adds_bos))
            self.default_add_eos = bool(self.config.get("add_eos_token", self.hf_adds_eos))

    def encode(self, text: str, add_bos: bool = True, add_eos: bool = True, **kwargs) -> list[int]:
        ids = self.tokenizer.encode(text, add_special_tokens=kwargs.get("add_special_tokens", True)).ids
        if add_bos and self.bos_id is not None and not self.hf_adds_bos:
            if not ids or ids[0] != self.bos_id:
                ids = [self.bos_id] + ids
        if add_eos and self.eos_id is not None and not self.hf_adds_eos:
            if not ids or ids[-1] != self.eos_id:
                ids = ids + [self.eos_id]
        return ids

    def decode(self, token_ids: list[int], skip_special_tokens: bool = True, **kwargs) -> str:
        return self.tokenizer.decode(token_ids, skip_special_tokens=skip_special_tokens)

    @property
    def vocab_size(self) -> int:
        return self.tokenizer.get_vocab_size()

    def get_vocab_size(self) -> int:
        return self.tokenizer.get_vocab_size()

    def get_vocab(self) -> dict[str, int]:
        return self.tokenizer.get_vocab()

    def token_to_id(self, token: str) -> int | None:
        return self.tokenizer.token_to_id(token)

    def id_to_token(self, token_id: int) -> str | None:
        return self.tokenizer.id_to_token(token_id)
