from torchtitan_b200.models.llama3 import model_registry  # the same model spec; the plan lives in the trainer

__all__ = ["model_registry"]
