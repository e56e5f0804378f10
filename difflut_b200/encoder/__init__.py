"""Encoders of the hot path: the thermometer encoder and its base class."""

from .base_encoder import BaseEncoder
from .thermometer import DistributiveThermometerEncoder, GaussianThermometerEncoder, ThermometerEncoder

__all__ = ["BaseEncoder", "ThermometerEncoder", "GaussianThermometerEncoder", "DistributiveThermometerEncoder"]
