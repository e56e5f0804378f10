"""Layers of the hot path (registered on import)."""

from .base_layer import BaseLUTLayer
from .layer_config import LayerConfig
from .learnable_layer import LearnableLayer
from .random_layer import RandomLayer

__all__ = ["BaseLUTLayer", "RandomLayer", "LearnableLayer", "LayerConfig"]
