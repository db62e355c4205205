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
        steps: int = -1
        """Held-out batches per validation run; -1 = until the (finite) validation loader is exhausted."""
        timesteps: int = 8
        """Evenly spaced noise levels at which the loss is evaluated for every batch (``all_timesteps``)."""
        all_timesteps: bool = True
        """Evaluate every sample at all ``timesteps`` levels. When False the loader deals one of the eight stratified
        levels to each sample in turn (the reference's default, torchtitan/models/flux/validate.py:60-61, 103-107)."""
        save_img_count: int = 0
        """Images sampled from the validation prompts per validation run (-1: one for every prompt seen)."""
        save_img_folder: str = "validation_images"
        dataloader: FluxDataLoader.Config = field(default_factory=lambda: FluxDataLoader.Config(dataset="coco-validation", generate_timesteps=True))

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
            import dataclasses

            dl = dataclasses.replace(config.dataloader, generate_timesteps=not config.all_timesteps,
                                     infinite=config.steps != -1)
            if config.steps == -1:
                from torchtitan_b200.tools.logging import logger

                logger.warning("Setting validation steps to -1 might cause hangs because of unequal sample counts across ranks "
                               "when dataset is exhausted.")
            self.dataloader = dl.build(dp_world_size=dp_world_size, dp_rank=dp_rank, local_batch_size=local_batch_size)
        self._tokenizers = None
        super().__init__(config)
        self.t, self.steps, self.n_t = trainer, config.steps, config.timesteps
        self.save_img_count, self.save_img_folder = config.save_img_count, config.save_img_folder
        self.metrics_processor = metrics_processor

    def attach(self, trainer) -> None:
        self.t = trainer

    def _prompt_tokenizers(self):
        """(t5, clip) tokenizers of the validation loader: sampling with guidance encodes the empty prompt with them."""
        if self._tokenizers is None:
            ds = getattr(self.dataloader, "dataset", None)
            self._tokenizers = (getattr(ds, "_t5", None), getattr(ds, "_clip", None))
            if self._tokenizers[0] is None:
                from .tokenizer import build_flux_tokenizer

                c, e = self.config.dataloader, self.config.dataloader.encoder
                self._tokenizers = build_flux_tokenizer(
                    t5_path=c.t5_tokenizer_path or e.t5_encoder, clip_path=c.clip_tokenizer_path or e.clip_encoder,
                    t5_max_length=c.t5_max_length, clip_max_length=c.clip_max_length, test_mode=c.test_tokenizer or e.test_mode)
        return self._tokenizers

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
        self._images_left, self._saved = self.save_img_count, 0
        done = 0
        while self.steps == -1 or done < self.steps:
            nxt = next(data_iterator, None)
            if nxt is None:
                break
            done += 1
            inputs, images = nxt
            given_t = inputs.pop("timestep", None) if isinstance(inputs, dict) else None
            batch = preprocess_data(tr.device, tr._dtype, autoencoder=tr.autoencoder, clip_encoder=tr.clip_encoder,
                                    t5_encoder=tr.t5_encoder, batch={**inputs, "image": images})
            x = batch["img_encodings"]
            bsz, _, lh, lw = x.shape
            img_ids = create_position_encoding_for_latents(bsz, lh, lw).to(tr.device)
            txt_ids = torch.zeros(bsz, batch["t5_encodings"].shape[1], 3, device=tr.device)
            # a loader built with ``generate_timesteps`` assigns one stratified noise level to every sample; otherwise
            # every batch is evaluated at all ``timesteps`` levels
            levels = [torch.as_tensor(given_t, dtype=torch.float32, device=tr.device).reshape(bsz)] if given_t is not None else \
                [torch.full((bsz,), (k + 0.5) / self.n_t, device=tr.device) for k in range(self.n_t)]
            for t in levels:
                noise = torch.randn_like(x)
                sig = t.view(-1, 1, 1, 1).to(x.dtype)
                with tr.maybe_enable_amp:
                    pred = model(img=pack_latents((1 - sig) * x + sig * noise), img_ids=img_ids, txt=batch["t5_encodings"],
                                 txt_ids=txt_ids, y=batch["clip_encodings"], timesteps=t.to(x.dtype))
                total += float(torch.nn.functional.mse_loss(pred.float(), pack_latents(noise - x).float()))
                count += 1
            budget = self._images_left
            if budget != 0:
                prompts = inputs.get("prompt") if isinstance(inputs, dict) else None
                n = images.shape[0] if budget < 0 else min(budget, images.shape[0])
                t5_tok, clip_tok = self._prompt_tokenizers()
                with tr.maybe_enable_amp:
                    imgs = generate_image(tr.device, tr._dtype, model=model, autoencoder=tr.autoencoder,
                                          clip_encoder=tr.clip_encoder, t5_encoder=tr.t5_encoder,
                                          clip_tokens=inputs["clip_tokens"][:n], t5_tokens=inputs["t5_tokens"][:n],
                                          clip_tokenizer=clip_tok, t5_tokenizer=t5_tok, job_config=tr.config,
                                          height=16 * (images.shape[-2] // 16), width=16 * (images.shape[-1] // 16))
                rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
                for i, im in enumerate(imgs):
                    save_image(im, os.path.join(tr.config.dump_folder, self.save_img_folder),
                               f"image_rank{rank}_{step}_{self._saved}.png", prompt=prompts[i] if prompts else None)
                    self._saved += 1
                if budget > 0:
                    self._images_left -= n
        model.train()
        return total / max(1, count)
