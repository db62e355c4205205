from dataclasses import dataclass

from torchtitan_b200.trainer import Trainer


@dataclass(kw_only=True, slots=True)
class TransformersBackendConfig(Trainer.Config):
    hf_model: str = ""
    """Hugging Face model id (e.g. ``Qwen/Qwen3-4B-Instruct-2507``); its ``config.json`` is read from
    ``<hf_assets_path>`` when present, otherwise the architecture defaults of the matching ``transformers`` config class
    are used (no network access is attempted)."""
