"""``Embedding`` with the Module protocol. Parity: torchtitan/models/common/embedding.py:16-52
(normal(0, 1) init)."""

from dataclasses import dataclass, field

import torch.nn as nn

from torchtitan_b200.protocols.module import Module


class Embedding(nn.Embedding, Module):
    @dataclass(kw_only=True, slots=True)
    class Config(Module.Config):
        num_embeddings: int = field(init=False)
        embedding_dim: int = field(init=False)
        init_mean: float = 0.0
        init_std: float = 1.0

    def __init__(self, config: Config):
        if not (hasattr(config, "num_embeddings") and hasattr(config, "embedding_dim")):
            raise TypeError(
                "Embedding.Config requires 'num_embeddings' and 'embedding_dim' to be set "
                "(use Config.build(num_embeddings=..., embedding_dim=...))."
            )
        super().__init__(config.num_embeddings, config.embedding_dim)
        self.config = config

    def init_weights(self, **kwargs) -> None:
        nn.init.normal_(self.weight, mean=self.config.init_mean, std=self.config.init_std)
