"""Model families. Each sub-package exposes ``model_registry(flavor) -> ModelSpec`` and a
``config_registry`` module whose functions return complete ``Trainer.Config`` objects."""

_supported_models = frozenset(["llama3", "llama4", "qwen3", "deepseek_v3", "gpt_oss", "flux"])
