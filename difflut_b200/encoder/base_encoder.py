"""Encoder base class: fit / encode / forward with the reference's contract
(difflut/encoder/base_encoder.py:18-137)."""

from abc import ABC, abstractmethod
from typing import Any, Union

import torch
import torch.nn as nn

DEFAULT_ENCODER_NUM_BITS: int = 3
DEFAULT_ENCODER_FLATTEN: bool = True


class BaseEncoder(nn.Module, ABC):
    """Continuous values -> binary features; `fit` first, then `encode` (or call the module)."""

    def __init__(self, num_bits: int = DEFAULT_ENCODER_NUM_BITS, flatten: bool = DEFAULT_ENCODER_FLATTEN) -> None:
        super().__init__()
        assert num_bits > 0, "num_bits must be positive"
        assert isinstance(flatten, bool), "flatten must be a boolean"
        self.num_bits = int(num_bits)
        self.flatten = flatten
        self._is_fitted = False

    @abstractmethod
    def fit(self, x: Any) -> "BaseEncoder":
        ...

    @abstractmethod
    def encode(self, x: Any) -> torch.Tensor:
        ...

    def forward(self, x: Any) -> torch.Tensor:
        return self.encode(x)

    def _to_tensor(self, x: Any) -> torch.Tensor:
        return x if isinstance(x, torch.Tensor) else torch.tensor(x)

    def _check_fitted(self) -> None:
        if not self._is_fitted:
            raise RuntimeError(
                f"{self.__class__.__name__} must be fitted before encoding. "
                "Call fit() first with your training data to compute encoding parameters. "
                "Example: encoder.fit(train_data).encode(test_data)"
            )

    @property
    def is_fitted(self) -> bool:
        return self._is_fitted

    def to(self, device: Union[str, torch.device]) -> "BaseEncoder":
        """Move every public tensor attribute (e.g. `thresholds`) to `device`."""
        for name in dir(self):
            if name.startswith("_"):
                continue
            try:
                attr = getattr(self, name)
            except Exception:
                continue
            if isinstance(attr, torch.Tensor):
                setattr(self, name, attr.to(device))
        return self

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(num_bits={self.num_bits}, flatten={self.flatten})"
