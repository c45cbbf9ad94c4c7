"""A B200-native inference engine for the Qwen2.5 dense decoder (single GPU)."""
from . import config, weights, cache  # noqa: F401

__version__ = "0.1.0"
