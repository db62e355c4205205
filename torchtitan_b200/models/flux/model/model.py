"""FLUX.1 flow-matching transformer (torchtitan/models/flux/model/model.py)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from torchtitan_b200.protocols.model import BaseModel

from .autoencoder import AutoEncoderParams
from .layers import DoubleStreamBlock, EmbedND, LastLayer, MLPEmbedder, SingleStreamBlock, timestep_embedding


class FluxModel(BaseModel):
    @dataclass(kw_only=True, slots=True)
    class Config(BaseModel.Config):
        in_channels: int = 64
        out_channels: int = 64
        vec_in_dim: int = 768
        context_in_dim: int = 512
        hidden_size: int = 3072
        mlp_ratio: float = 4.0
        num_heads: int = 24
        depth: int = 19
        depth_single_blocks: int = 38
        axes_dim: tuple = (16, 56, 56)
        theta: int = 10_000
        qkv_bias: bool = True
        autoencoder_params: AutoEncoderParams = field(default_factory=AutoEncoderParams)

        def update_from_config(self, *, trainer_config, **kwargs) -> None:
            par = trainer_config.parallelism
            if par.tensor_parallel_degree > 1 or par.pipeline_parallel_degree > 1:
                raise NotImplementedError("FLUX supports FSDP / HSDP / context parallel only")

        def get_nparams_and_flops(self, model: nn.Module, seq_len: int):
            n = sum(p.numel() for p in model.parameters())
            return n, 6 * n + 12 * (self.depth + self.depth_single_blocks) * self.hidden_size * seq_len

    def __init__(self, config: Config):
        super().__init__()
        c = self.config = config
        if c.hidden_size % c.num_heads:
            raise ValueError(f"Hidden size {c.hidden_size} must be divisible by num_heads {c.num_heads}")
        pe_dim = c.hidden_size // c.num_heads
        if sum(c.axes_dim) != pe_dim:
            raise ValueError(f"Got {c.axes_dim} but expected positional dim {pe_dim}")
        self.hidden_size, self.num_heads = c.hidden_size, c.num_heads
        self.pe_embedder = EmbedND(pe_dim, c.theta, c.axes_dim)
        self.img_in = nn.Linear(c.in_channels, c.hidden_size)
        self.time_in = MLPEmbedder(256, c.hidden_size)
        self.vector_in = MLPEmbedder(c.vec_in_dim, c.hidden_size)
        self.txt_in = nn.Linear(c.context_in_dim, c.hidden_size)
        self.double_blocks = nn.ModuleList(DoubleStreamBlock(c.hidden_size, c.num_heads, c.mlp_ratio, c.qkv_bias) for _ in range(c.depth))
        self.single_blocks = nn.ModuleList(SingleStreamBlock(c.hidden_size, c.num_heads, c.mlp_ratio) for _ in range(c.depth_single_blocks))
        self.final_layer = LastLayer(c.hidden_size, 1, c.out_channels)

    def init_weights(self, **kwargs):
        for m in (self.img_in, self.txt_in):
            nn.init.xavier_uniform_(m.weight)
            nn.init.zeros_(m.bias)
        self.time_in.init_weights()
        self.vector_in.init_weights()
        for b in list(self.double_blocks) + list(self.single_blocks):
            b.init_weights()
        self.final_layer.init_weights()

    def forward(self, img, img_ids, txt, txt_ids, timesteps, y):
        if img.ndim != 3 or txt.ndim != 3:
            raise ValueError("Input img and txt tensors must have 3 dimensions.")
        img = self.img_in(img)
        vec = self.time_in(timestep_embedding(timesteps, 256).to(img.dtype)) + self.vector_in(y)
        txt = self.txt_in(txt)
        pe = self.pe_embedder(torch.cat((txt_ids, img_ids), dim=1))
        for block in self.double_blocks:
            img, txt = block(img=img, txt=txt, vec=vec, pe=pe)
        x = torch.cat((txt, img), 1)
        for block in self.single_blocks:
            x = block(x, vec=vec, pe=pe)
        return self.final_layer(x[:, txt.shape[1] :], vec)
