"""Validation for FLUX: flow-matching loss at fixed, evenly spaced timesteps on held-out batches, optionally sampling a few
images and saving them as PNG files (torchtitan/models/flux/validate.py)."""

from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch

from torchtitan_b200.components.validate import BaseValidator

from .flux_datasets import FluxDataLoader
from .inference.sampling import generate_image, save_image
from .utils import create_position_encoding_for_latents, pack_latents, preprocess_data


class FluxValidator(BaseValidator):
    """Built from the job configuration (``--validator.enable``) like the text validator; ``attach(trainer)`` hands it the
    frozen encoders and the autoencoder once the trainer owns them."""

    @dataclass(kw_only=True, slots=True)
    class Config(BaseValidator.Config):
        enable: bool = False
        steps: int = 4
        """Held-out batches per validation run."""
        timesteps: int = 8
        """Evenly spaced noise levels at which the loss is evaluated for every batch."""
        save_img_count: int = 0
        save_img_folder: str = "img"
        dataloader: FluxDataLoader.Config = field(default_factory=lambda: FluxDataLoader.Config(dataset="synthetic"))

    def __init__(self, config=None, trainer=None, steps: int = 4, timesteps: int = 8, save_img_count: int = 0,
                 save_img_folder: str = "img", *, dp_world_size: int = 1, dp_rank: int = 0, local_batch_size: int = 1,
                 metrics_processor=None, **kwargs):
        if config is not None and not isinstance(config, FluxValidator.Config):      # positional use: FluxValidator(trainer, ...)
            trainer, config = config, None
        if config is None:
            config = FluxValidator.Config(steps=steps, timesteps=timesteps, save_img_count=save_img_count,
                                          save_img_folder=save_img_folder)
            self.dataloader = None
        else:
            self.dataloader = config.dataloader.build(dp_world_size=dp_world_size, dp_rank=dp_rank, local_batch_size=local_batch_size)
        super().__init__(config)
        self.t, self.steps, self.n_t = trainer, config.steps, config.timesteps
        self.save_img_count, self.save_img_folder = config.save_img_count, config.save_img_folder
        self.metrics_processor = metrics_processor

    def attach(self, trainer) -> None:
        self.t = trainer

    def validate(self, model_parts_or_iterator, step: int) -> float:
        """Trainer protocol: ``validate(model_parts, step)`` draws from the validator's own loader and logs the loss;
        ``validate(iterator, step)`` evaluates on the given batches and returns the loss."""
        if isinstance(model_parts_or_iterator, (list, tuple)):
            loss = self._validate(iter(self.dataloader), step)
            if self.t.parallel_dims.dp_enabled:
                from torchtitan_b200.parallel import utils as dist_utils

                loss = float(dist_utils.dist_mean(torch.tensor(loss, device=self.t.device), self.t.parallel_dims.get_mesh("batch")))
            if self.metrics_processor is not None:
                self.metrics_processor.log_validation(loss=loss, step=step)
            return loss
        return self._validate(model_parts_or_iterator, step)

    @torch.no_grad()
    def _validate(self, data_iterator, step: int) -> float:
        tr = self.t
        model = tr.model_parts[0]
        model.eval()
        total, count = 0.0, 0
        for _ in range(self.steps):
            inputs, images = next(data_iterator)
            batch = preprocess_data(tr.device, tr._dtype, autoencoder=tr.autoencoder, clip_encoder=tr.clip_encoder,
                                    t5_encoder=tr.t5_encoder, batch={**inputs, "image": images})
            x = batch["img_encodings"]
            bsz, _, lh, lw = x.shape
            img_ids = create_position_encoding_for_latents(bsz, lh, lw).to(tr.device)
            txt_ids = torch.zeros(bsz, batch["t5_encodings"].shape[1], 3, device=tr.device)
            for k in range(self.n_t):
                t = torch.full((bsz,), (k + 0.5) / self.n_t, device=tr.device)
                noise = torch.randn_like(x)
                sig = t.view(-1, 1, 1, 1).to(x.dtype)
                pred = model(img=pack_latents((1 - sig) * x + sig * noise), img_ids=img_ids, txt=batch["t5_encodings"], txt_ids=txt_ids,
                             y=batch["clip_encodings"], timesteps=t.to(x.dtype))
                total += float(torch.nn.functional.mse_loss(pred.float(), pack_latents(noise - x).float()))
                count += 1
            if self.save_img_count:
                imgs = generate_image(tr.device, tr._dtype, model=model, autoencoder=tr.autoencoder, clip_encoder=tr.clip_encoder,
                                      t5_encoder=tr.t5_encoder, clip_tokens=inputs["clip_tokens"][: self.save_img_count],
                                      t5_tokens=inputs["t5_tokens"][: self.save_img_count], height=images.shape[-2], width=images.shape[-1])
                for i, im in enumerate(imgs):
                    save_image(im, os.path.join(tr.config.dump_folder, self.save_img_folder), f"step{step}_img{i}.png")
        model.train()
        return total / max(1, count)
