"""Architectures: each module turns its typed configuration into a ModelSpec and registers itself."""
from . import llama4  # noqa: F401
