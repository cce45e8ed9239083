"""Importing this package registers the architectures the engine ships with."""
from . import llama  # noqa: F401
