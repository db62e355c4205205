"""FLUX job configurations (torchtitan/models/flux/config_registry.py:24-195: the same batch sizes, step counts,
guidance probability, sampling and validation settings).

``flux_debugmodel`` runs without any downloaded asset: the image-caption shard under ``tests/assets/cc12m_test``
(``--dataloader.dataset synthetic`` needs no files at all), the asset-free tokenizer when the tokenizer folders are
absent, and randomly initialised encoders of the model's input widths (``--encoder.random_init False`` loads the
checkpoints the ``--encoder.*`` fields name)."""

from torchtitan_b200.components.checkpoint import CheckpointManager
from torchtitan_b200.components.lr_scheduler import LRSchedulersContainer
from torchtitan_b200.components.metrics import MetricsProcessor
from torchtitan_b200.components.optimizer import OptimizersContainer
from torchtitan_b200.config import ActivationCheckpointConfig, TrainingConfig

from . import model_registry
from .configs import Encoder, Inference, Validation
from .flux_datasets import FluxDataLoader
from .trainer import FluxTrainer
from .validate import FluxValidator

_AE = "assets/hf/FLUX.1-dev/ae.safetensors"


def flux_debugmodel() -> FluxTrainer.Config:
    encoder = Encoder(t5_encoder="google/t5-v1_1-xxl", clip_encoder="openai/clip-vit-large-patch14", max_t5_encoding_len=256,
                      autoencoder_path=_AE, random_init=True)
    return FluxTrainer.Config(
        hf_assets_path="tests/assets/tokenizer", metrics=MetricsProcessor.Config(log_freq=1),
        model_spec=model_registry("flux-debug"), tokenizer=None,
        dataloader=FluxDataLoader.Config(dataset="cc12m-test", classifier_free_guidance_prob=0.447, img_size=256, encoder=encoder,
                                         hf_assets_path="tests/assets/tokenizer"),
        optimizer=OptimizersContainer.Config(lr=8e-4), lr_scheduler=LRSchedulersContainer.Config(warmup_steps=1, decay_ratio=0.0),
        training=TrainingConfig(local_batch_size=4, steps=10, max_norm=2.0),
        encoder=encoder, checkpoint=CheckpointManager.Config(interval=10, last_save_model_only=False),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
        validation=Validation(enable_classifier_free_guidance=True, classifier_free_guidance_scale=5.0, denoising_steps=4),
        validator=FluxValidator.Config(
            freq=5, steps=48, all_timesteps=False, save_img_count=1, save_img_folder="img",
            dataloader=FluxDataLoader.Config(dataset="cc12m-test", classifier_free_guidance_prob=0.447, img_size=256,
                                             generate_timesteps=True, encoder=encoder)),
        inference=Inference(save_img_folder="inference_results",
                            prompts_path="./torchtitan_b200/models/flux/inference/prompts.txt", local_batch_size=2),
    )


def _full(flavor: str, *, batch: int, t5_len: int, val_steps: int) -> FluxTrainer.Config:
    encoder = Encoder(t5_encoder="google/t5-v1_1-xxl", clip_encoder="openai/clip-vit-large-patch14", max_t5_encoding_len=t5_len,
                      autoencoder_path=_AE)
    return FluxTrainer.Config(
        metrics=MetricsProcessor.Config(log_freq=100), model_spec=model_registry(flavor), tokenizer=None,
        dataloader=FluxDataLoader.Config(dataset="cc12m-wds", classifier_free_guidance_prob=0.447, img_size=256,
                                         t5_max_length=t5_len, encoder=encoder),
        optimizer=OptimizersContainer.Config(lr=1e-4), lr_scheduler=LRSchedulersContainer.Config(warmup_steps=3000, decay_ratio=0.0),
        training=TrainingConfig(local_batch_size=batch, steps=30000),
        encoder=encoder, checkpoint=CheckpointManager.Config(interval=1000),
        activation_checkpoint=ActivationCheckpointConfig(mode="full"),
        validation=Validation(enable_classifier_free_guidance=True, classifier_free_guidance_scale=5.0, denoising_steps=50),
        validator=FluxValidator.Config(
            freq=1000, steps=val_steps, all_timesteps=False, save_img_count=50, save_img_folder="img",
            dataloader=FluxDataLoader.Config(dataset="coco-validation", classifier_free_guidance_prob=0.0, img_size=256,
                                             t5_max_length=t5_len, generate_timesteps=True, encoder=encoder)),
    )


def flux_dev() -> FluxTrainer.Config:
    return _full("flux-dev", batch=32, t5_len=512, val_steps=12)


def flux_schnell() -> FluxTrainer.Config:
    return _full("flux-schnell", batch=64, t5_len=256, val_steps=6)
