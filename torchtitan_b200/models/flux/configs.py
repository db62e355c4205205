"""Configuration sections of the FLUX trainer beside the common ones (torchtitan/models/flux/configs.py:10-53):
``--encoder.*`` (frozen text encoders and autoencoder), ``--validation.*`` (how validation images are sampled) and
``--inference.*`` (the prompt-file inference entry point)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(kw_only=True, slots=True)
class Encoder:
    t5_encoder: str = "google/t5-v1_1-small"
    """T5 encoder: a local folder (Hugging Face layout) or a hub name."""
    clip_encoder: str = "openai/clip-vit-large-patch14"
    """CLIP text encoder: a local folder or a hub name."""
    autoencoder_path: str = "assets/hf/FLUX.1-dev/ae.safetensors"
    """Autoencoder weights (safetensors)."""
    max_t5_encoding_len: int = 256
    """Length the T5 token rows are padded / truncated to."""
    test_mode: bool = False
    """Integration-test mode: small randomly initialised encoders and the asset-free tokenizer."""
    random_init: bool = False
    """Randomly initialised encoders / autoencoder of the real architecture sizes given by the model (offline runs);
    ``test_mode`` implies it."""
    hidden: int = 64

    @property
    def offline(self) -> bool:
        return self.test_mode or self.random_init


@dataclass(kw_only=True, slots=True)
class Validation:
    enable_classifier_free_guidance: bool = False
    """Sample with classifier-free guidance (two forward passes per step, batched)."""
    classifier_free_guidance_scale: float = 5.0
    denoising_steps: int = 50
    """Euler steps per generated image."""
    eval_freq: int = 100
    """Sampling frequency during training."""


@dataclass(kw_only=True, slots=True)
class Inference:
    save_img_folder: str = "inference_results"
    """Folder under the dump folder that receives the images."""
    prompts_path: str = "./torchtitan_b200/models/flux/inference/prompts.txt"
    """Text file with one prompt per line."""
    local_batch_size: int = 2
    img_size: int = 256
