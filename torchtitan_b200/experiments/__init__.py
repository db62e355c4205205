"""Experiments built on the core framework (one-way dependency: core never imports these)."""

_supported_experiments = frozenset(["rl", "ft", "forge", "graph_trainer", "vlm", "transformers_modeling_backend", "autoparallel"])
