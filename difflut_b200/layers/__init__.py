"""Layers of the hot path (registered on import)."""

from .base_layer import BaseLUTLayer
from .convolutional import ConvolutionalLayer, ConvolutionConfig
from .layer_config import GroupedInputConfig, LayerConfig
from .learnable_layer import LearnableLayer
from .random_layer import RandomLayer
from .stack import DWNStack

__all__ = ["BaseLUTLayer", "RandomLayer", "LearnableLayer", "ConvolutionalLayer", "ConvolutionConfig",
           "LayerConfig", "GroupedInputConfig", "DWNStack"]
