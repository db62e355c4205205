"""``--module graph_trainer`` entry: re-exports the per-model configurations."""

from .deepseek_v3.config_registry import *  # noqa: F401,F403
from .llama3.config_registry import *  # noqa: F401,F403
