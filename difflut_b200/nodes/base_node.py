"""Base class of LUT nodes: validation, train/eval dispatch, regularizers, bitstream export.

Behaviour follows difflut/nodes/base_node.py:22-371 (same defaults, exception types and
warnings).  A node maps (batch, input_dim) -> (batch, output_dim).
"""

import itertools
import warnings
from abc import ABC, abstractmethod
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..utils.warnings import warn_default_value

DEFAULT_NODE_INPUT_DIM: int = 6
DEFAULT_NODE_OUTPUT_DIM: int = 1
NODE_INPUT_DIM_WARNING_THRESHOLD: int = 10
NODE_OUTPUT_DIM_WARNING_THRESHOLD: int = 10


def validate_node_dims(input_dim, output_dim, stacklevel: int = 3) -> Tuple[int, int]:
    """Defaults, type/range checks and size warnings shared by nodes and stacked layers."""
    if input_dim is None:
        input_dim = DEFAULT_NODE_INPUT_DIM
        warn_default_value("input_dim", input_dim, stacklevel=stacklevel)
    if output_dim is None:
        output_dim = DEFAULT_NODE_OUTPUT_DIM
        warn_default_value("output_dim", output_dim, stacklevel=stacklevel)
    if not isinstance(input_dim, int) or input_dim <= 0:
        raise ValueError(f"input_dim must be a positive integer, but got {input_dim}. Example: input_dim=6")
    if input_dim > NODE_INPUT_DIM_WARNING_THRESHOLD:
        warnings.warn(
            f"input_dim={input_dim} is quite large. LUT nodes with >{NODE_INPUT_DIM_WARNING_THRESHOLD} inputs "
            f"need 2^{input_dim} table entries each.",
            UserWarning,
            stacklevel=stacklevel,
        )
    if not isinstance(output_dim, int) or output_dim <= 0:
        raise ValueError(f"output_dim must be a positive integer, but got {output_dim}. Example: output_dim=1")
    if output_dim > NODE_OUTPUT_DIM_WARNING_THRESHOLD:
        warnings.warn(
            f"output_dim={output_dim} is quite large. This may increase memory requirements significantly.",
            UserWarning,
            stacklevel=stacklevel,
        )
    return input_dim, output_dim


def validate_regularizers(regularizers) -> Dict[str, list]:
    """Each entry must be [callable, numeric weight, dict kwargs]."""
    if not regularizers:
        return {}
    checked = {}
    for name, value in regularizers.items():
        if not isinstance(value, (list, tuple)):
            raise ValueError(
                f"Regularizer '{name}' must be a list/tuple of [function, weight, kwargs], "
                f"but got {type(value).__name__}."
            )
        if len(value) != 3:
            raise ValueError(
                f"Regularizer '{name}' must have exactly 3 elements [function, weight, kwargs], "
                f"but got {len(value)} elements."
            )
        fn, weight, kwargs = value
        if not callable(fn):
            raise TypeError(f"Regularizer '{name}' function must be callable, but got {type(fn).__name__}.")
        if not isinstance(weight, (int, float)):
            raise TypeError(f"Regularizer '{name}' weight must be numeric, but got {type(weight).__name__}.")
        if not isinstance(kwargs, dict):
            raise TypeError(f"Regularizer '{name}' kwargs must be a dict, but got {type(kwargs).__name__}.")
        checked[name] = [fn, weight, kwargs]
    return checked


class BaseNode(nn.Module, ABC):
    def __init__(
        self,
        input_dim: Optional[int] = None,
        output_dim: Optional[int] = None,
        regularizers: Optional[Dict[str, Tuple[Callable, float, Dict[str, Any]]]] = None,
        init_fn: Optional[Callable[[torch.Tensor], None]] = None,
        init_kwargs: Optional[Dict[str, Any]] = None,
        **kwargs,  # accepted and ignored, as in the reference
    ) -> None:
        super().__init__()
        self.input_dim, self.output_dim = validate_node_dims(input_dim, output_dim, stacklevel=3)
        self.regularizers = {} if regularizers is None else regularizers
        if init_fn is not None and not callable(init_fn):
            raise TypeError(
                f"init_fn must be callable, but got {type(init_fn).__name__}. "
                f"Signature should be: init_fn(parameter: torch.Tensor, **kwargs) -> None"
            )
        self.init_fn = init_fn
        self.init_kwargs = {} if init_kwargs is None else init_kwargs
        if not isinstance(self.init_kwargs, dict):
            raise TypeError(f"init_kwargs must be a dict, but got {type(self.init_kwargs).__name__}")
        self.regularizers = validate_regularizers(self.regularizers)

    @property
    def num_inputs(self) -> int:
        return self.input_dim

    @property
    def num_outputs(self) -> int:
        return self.output_dim

    def _apply_init_fn(self, param: torch.Tensor, name: str = "parameter") -> None:
        if self.init_fn is None:
            return
        try:
            self.init_fn(param, **self.init_kwargs)
        except Exception as e:
            raise RuntimeError(
                f"Initialization of '{name}' failed with error: {e}. "
                f"Check that init_fn is compatible with the parameter and init_kwargs are correct."
            )

    @abstractmethod
    def forward_train(self, x: torch.Tensor) -> torch.Tensor:
        ...

    def forward_eval(self, x: torch.Tensor) -> torch.Tensor:
        return (self.forward_train(x) > 0.5).float()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_train(x) if self.training else self.forward_eval(x)

    def forward_with_mapping(self, x: torch.Tensor, mapping_indices: torch.Tensor) -> torch.Tensor:
        """(B, input_size) + (layer_size, input_dim) indices -> node applied to the gathered inputs."""
        rows = torch.arange(x.shape[0], device=x.device).view(-1, 1, 1)
        return self.forward(x[rows, mapping_indices])

    def regularization(self) -> torch.Tensor:
        reg = self._builtin_regularization()
        for name, (fn, weight, kwargs) in self.regularizers.items():
            try:
                reg = reg + weight * fn(self, **kwargs)
            except Exception as e:
                raise RuntimeError(
                    f"Regularizer '{name}' failed with error: {e}. "
                    f"Check that the regularizer function is correct and compatible with the node."
                )
        return reg

    def _param_device(self) -> torch.device:
        for p in self.parameters():
            return p.device
        return torch.device("cpu")

    def _builtin_regularization(self) -> torch.Tensor:
        return torch.tensor(0.0, device=self._param_device())

    def export_bitstream(self) -> List[int]:
        """Output bits of `forward_eval` on all 2^n input patterns (first input = slowest digit)."""
        with torch.no_grad():
            pats = torch.tensor(list(itertools.product([0, 1], repeat=self.num_inputs)),
                                dtype=torch.float32, device=self._param_device())
            out = self.forward_eval(pats)
        return [int(v > 0.5) for v in out.flatten().tolist()]
