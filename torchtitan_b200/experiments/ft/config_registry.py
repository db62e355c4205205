"""``--module ft`` entry: re-exports the fault-tolerant job configurations."""

from .llama3.config_registry import llama3_ft_debugmodel  # noqa: F401
