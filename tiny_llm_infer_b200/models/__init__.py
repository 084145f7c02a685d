"""Architectures.  Importing this package registers them (see ``config.base``)."""
from . import qwen3  # noqa: F401
from .model import Model, expected_tensors
