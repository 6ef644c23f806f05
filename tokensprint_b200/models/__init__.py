"""Architectures.  Importing this package registers them (config/registry.py)."""

from tokensprint_b200.models import dazilix, fegetar, pekunex, qwen3, vasosun  # noqa: F401
