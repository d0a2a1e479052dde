"""Architectures this engine builds.  Importing a module registers its architecture name."""
from . import qwen3  # noqa: F401
