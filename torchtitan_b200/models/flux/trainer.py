"""``FluxTrainer``: flow-matching training step on top of the base trainer.

Parity: torchtitan/models/flux/trainer.py:26-285 -- frozen T5 / CLIP encoders and autoencoder are built beside the model;
a step encodes the batch (no grad), draws noise and a uniform time per sample, forms ``x_t = (1 - t) x + t eps``, and
regresses the packed velocity ``eps - x`` with a sum-of-squares loss divided by the global number of latent elements."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from torchtitan_b200.parallel import utils as dist_utils
from torchtitan_b200.trainer import Trainer

from .configs import Encoder, Inference, Validation
from .model.autoencoder import load_ae
from .model.hf_embedder import FluxEmbedder
from .utils import create_position_encoding_for_latents, pack_latents, preprocess_data
from .validate import FluxValidator


class FluxTrainer(Trainer):
    @dataclass(kw_only=True, slots=True)
    class Config(Trainer.Config):
        encoder: Encoder = field(default_factory=Encoder)
        validation: Validation = field(default_factory=Validation)
        inference: Inference = field(default_factory=Inference)
        validator: FluxValidator.Config = field(default_factory=FluxValidator.Config)

    def __init__(self, config: Config):
        super().__init__(config)
        from torchtitan_b200.config import TORCH_DTYPE_MAP

        # dtype of the frozen encoders and of their outputs: the mixed-precision parameter dtype when FSDP casts the
        # model's parameters to it, float32 otherwise (then autocast, if any, does the casting inside the model)
        self._dtype = (TORCH_DTYPE_MAP[config.training.mixed_precision_param]
                       if self.device.type == "cuda" and self.parallel_dims.fsdp_enabled else torch.float32)
        e = config.encoder
        self.autoencoder = load_ae(e.autoencoder_path, self.model_config.autoencoder_params, device=self.device, dtype=self._dtype,
                                   random_init=e.offline)
        self.clip_encoder = FluxEmbedder(e.clip_encoder, random_init=e.offline, hidden=self.model_config.vec_in_dim).to(self.device, self._dtype)
        self.t5_encoder = FluxEmbedder(e.t5_encoder, random_init=e.offline, hidden=self.model_config.context_in_dim).to(self.device, self._dtype)
        # Noise and noise levels must differ between data-parallel ranks (they see different images) and agree between
        # the ranks that share a batch (context parallel): a generator of their own, seeded by the job's base seed and
        # the data-parallel rank. The reference gets the same effect from distinct global seeds along the fsdp and
        # dp_replicate mesh dimensions (torchtitan/models/flux/trainer.py:36-44).
        self._noise_gen = torch.Generator(device=self.device)
        self._noise_gen.manual_seed((int(self.base_seed) + 1_000_003 * (self.dp_rank + 1)) % 2**63)
        if self.validator is not None:
            self.validator.attach(self)

    def forward_backward_step(self, *, input_dict, labels, global_valid_tokens=None):
        input_dict = dict(input_dict)
        input_dict["image"] = labels
        batch = preprocess_data(self.device, self._dtype, autoencoder=self.autoencoder, clip_encoder=self.clip_encoder,
                                t5_encoder=self.t5_encoder, batch=input_dict)
        target_latents = batch["img_encodings"]
        n_local = torch.tensor(float(target_latents.numel()), device=self.device)
        n_global = dist_utils.dist_sum(n_local, self.parallel_dims.get_mesh("batch")) if self.parallel_dims.dp_enabled else n_local
        bsz, _, lh, lw = target_latents.shape
        with torch.no_grad():
            noise = torch.randn(target_latents.shape, dtype=target_latents.dtype, device=self.device, generator=self._noise_gen)
            t = torch.rand(bsz, device=self.device, generator=self._noise_gen)
            sig = t.view(-1, 1, 1, 1).to(target_latents.dtype)
            latents = pack_latents((1 - sig) * target_latents + sig * noise)
            target = pack_latents(noise - target_latents)
            img_ids = create_position_encoding_for_latents(bsz, lh, lw).to(self.device)
            txt_ids = torch.zeros(bsz, batch["t5_encodings"].shape[1], 3, device=self.device)
        with self.train_context(), self.maybe_enable_amp:
            pred = self.model_parts[0](img=latents, img_ids=img_ids, txt=batch["t5_encodings"], txt_ids=txt_ids,
                                       y=batch["clip_encodings"], timesteps=t.to(latents.dtype))
            loss = self.loss_fn(pred, target) / n_global
        loss.backward()
        return loss

    def train_step(self, data_iterator) -> None:
        self.optimizers.zero_grad()
        losses = []
        for _ in range(self.gradient_accumulation_steps):
            input_dict, labels = next(data_iterator)
            losses.append(self.forward_backward_step(input_dict=input_dict, labels=labels).detach())
        grad_norm = dist_utils.clip_grad_norm_([p for m in self.model_parts for p in m.parameters()], self.config.training.max_norm,
                                               foreach=True, pp_mesh=None)
        self.checkpointer.maybe_wait_for_staging()
        self.optimizers.step()
        self.lr_schedulers.step()
        self.last_loss = torch.stack(losses).sum()
        self.last_grad_norm = grad_norm
        if self.metrics_processor.should_log(self.step):
            loss = self.last_loss
            if self.parallel_dims.dp_enabled:
                loss = dist_utils.dist_sum(loss, self.parallel_dims.get_mesh("batch"))
            self.metrics_processor.log(self.step, float(loss), float(loss), float(grad_norm))
