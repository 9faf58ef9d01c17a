"""Architectures.  Importing this package registers them (see ``config.base``)."""
from . import kaketar, panolorn, pevolorn, qwen3, tetodra  # noqa: F401
from .model import Model, expected_tensors
