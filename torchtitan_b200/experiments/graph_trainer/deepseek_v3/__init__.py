from torchtitan_b200.models.deepseek_v3 import model_registry

__all__ = ["model_registry"]
