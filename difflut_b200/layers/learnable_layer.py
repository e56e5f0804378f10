"""LearnableLayer: trainable soft connectivity (training) / argmax connectivity (eval).

Constructor, tau schedule, caching and accessors follow difflut/layers/learnable_layer.py:173-486:
training computes `x @ softmax(W/tau, -1).T` with W of shape (N*n, input_size) (row j*n+i feeds
slot i of node j); eval selects `argmax(W, -1)` (cached until the next `train()`), which turns
the layer into a fixed-connectivity layer that runs the RandomLayer kernels.
"""

import warnings
from typing import Optional, Type

import torch
import torch.nn as nn

from ..nodes.node_config import NodeConfig
from ..registry import register_layer
from ..utils.warnings import warn_default_value
from .base_layer import BaseLUTLayer
from .fused_ops import dwn_layer_eval
from .layer_config import LayerConfig
from .soft_select import soft_select

DEFAULT_LEARNABLE_LAYER_TAU: float = 0.001
DEFAULT_LEARNABLE_LAYER_TAU_START: float = 1.0
DEFAULT_LEARNABLE_LAYER_TAU_MIN: float = 0.0001
DEFAULT_LEARNABLE_LAYER_TAU_DECAY_ITERS: float = 1000.0
DEFAULT_LEARNABLE_LAYER_USE_CUDA_SOFT: bool = False
LEARNABLE_LAYER_CONNECTION_WARNING_THRESHOLD: int = 10
FAST_PATH_MAX_N: int = 6


class LearnableMappingModule(nn.Module):
    """Owns W (N*n, input_size); soft selection in training, cached hard selection in eval."""

    def __init__(self, input_size: int, output_size: int, tau: float = DEFAULT_LEARNABLE_LAYER_TAU,
                 use_cuda_soft: bool = DEFAULT_LEARNABLE_LAYER_USE_CUDA_SOFT):
        super().__init__()
        self.input_size = input_size
        self.output_size = output_size  # N*n selections
        self.tau = tau
        self.use_cuda_soft = use_cuda_soft
        self.W = nn.Parameter(torch.randn(output_size, input_size))
        nn.init.xavier_uniform_(self.W)
        self.register_buffer("_cached_hard_indices", None)
        self.register_buffer("_cached_hard_mask", None)
        self._cache_valid = False

    def train(self, mode: bool = True):
        was_training = self.training
        super().train(mode)
        if mode and not was_training:
            self._cache_valid = False
        return self

    def _compute_hard_selection(self) -> None:
        with torch.no_grad():
            self._cached_hard_indices = torch.argmax(self.W, dim=-1).int()

    def hard_indices(self) -> torch.Tensor:
        if not self._cache_valid or self._cached_hard_indices is None:
            self._compute_hard_selection()
            self._cache_valid = True
        return self._cached_hard_indices

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.training:
            return soft_select(x, self.W, self.tau)
        idx = self.hard_indices()
        return x[:, idx.long()]


@register_layer("learnable")
class LearnableLayer(BaseLUTLayer):
    def __init__(
        self,
        input_size: int,
        output_size: int,
        node_type: Type[nn.Module],
        node_kwargs: NodeConfig,
        tau: Optional[float] = None,
        tau_start: Optional[float] = None,
        tau_min: Optional[float] = None,
        tau_decay_iters: Optional[float] = None,
        layer_config: Optional[LayerConfig] = None,
        flip_probability: Optional[float] = None,
        grad_stabilization: Optional[str] = None,
        grad_target_std: Optional[float] = None,
        grad_subtract_mean: Optional[bool] = None,
        grad_epsilon: Optional[float] = None,
        use_cuda_soft: Optional[bool] = None,
    ):
        if tau is None:
            tau = DEFAULT_LEARNABLE_LAYER_TAU
            warn_default_value("tau", tau, stacklevel=2)
        if tau_start is None:
            tau_start = DEFAULT_LEARNABLE_LAYER_TAU_START
            warn_default_value("tau_start", tau_start, stacklevel=2)
        if tau_min is None:
            tau_min = DEFAULT_LEARNABLE_LAYER_TAU_MIN
            warn_default_value("tau_min", tau_min, stacklevel=2)
        if tau_decay_iters is None:
            tau_decay_iters = DEFAULT_LEARNABLE_LAYER_TAU_DECAY_ITERS
            warn_default_value("tau_decay_iters", tau_decay_iters, stacklevel=2)
        if use_cuda_soft is None:
            use_cuda_soft = DEFAULT_LEARNABLE_LAYER_USE_CUDA_SOFT
            warn_default_value("use_cuda_soft", use_cuda_soft, stacklevel=2)
        if tau_start < tau_min:
            warnings.warn(
                f"LearnableLayer: tau_start ({tau_start}) is less than tau_min ({tau_min}). "
                f"This means tau will be clamped immediately. Set tau_start >= tau_min.",
                UserWarning,
                stacklevel=2,
            )
        super().__init__(input_size, output_size, node_type, node_kwargs, layer_config, flip_probability,
                         grad_stabilization, grad_target_std, grad_subtract_mean, grad_epsilon)
        total = output_size * self.n
        if total > input_size * LEARNABLE_LAYER_CONNECTION_WARNING_THRESHOLD:
            warnings.warn(
                f"LearnableLayer: Creating {total} learnable connections from {input_size} inputs. "
                f"This may lead to overfitting.",
                UserWarning,
                stacklevel=2,
            )
        self.tau_start = tau_start
        self.tau_min = tau_min
        self.tau_decay_iters = tau_decay_iters
        self.tau = tau_start  # the reference starts from tau_start and ignores `tau` (learnable_layer.py:383)
        self.use_cuda_soft = use_cuda_soft
        self.mapping = LearnableMappingModule(input_size, output_size * self.n, self.tau, use_cuda_soft)

    def get_mapping(self, x: torch.Tensor) -> torch.Tensor:
        return self.mapping(x).view(x.shape[0], self.output_size, self.n)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._validate_input_dims(x)
        if not self.training and self._stacked == "dwn" and self.n <= FAST_PATH_MAX_N:
            idx = self.mapping.hard_indices().view(self.output_size, self.n)
            return dwn_layer_eval(x, self.luts, self._plan_for(idx, x.device, "hard"))
        if not self.training and self._stacked in ("dwn_stable", "hybrid"):
            idx = self.mapping.hard_indices().view(self.output_size, self.n)
            return dwn_layer_eval(x, self.stable_tables(), self._plan_for(idx, x.device, "hard"))
        if (self.training and self._stacked in ("dwn", "dwn_stable") and self.n <= FAST_PATH_MAX_N
                and x.shape[0] % 128 == 0):
            return self._forward_feature_major(x)
        return self._run_nodes(self.get_mapping(x))

    def _forward_feature_major(self, x: torch.Tensor) -> torch.Tensor:
        """Training with DWN-type nodes: the soft selection is contracted with swapped operands, so the
        selected values arrive feature-major (N*n, B), which is what the node kernels read, and their
        gradient leaves in the layout the weight-gradient contraction reads.  Same arithmetic as
        `_run_nodes(get_mapping(x))`."""
        from ..nodes.dwn_node import _identity_plan
        from .fused_ops import DWNLayerFunction, FeatureMajorInput
        from .soft_select import soft_select_t

        # the identity plan is disjoint (one reader per selected value) and with one output per node the plan's
        # virtual nodes are its nodes: the node kernel can then hand the gradient over as bf16 (see FeatureMajorInput)
        # the node kernels only read `selected value >= 0.5`: the contraction's epilogue packs those bits itself
        channel = FeatureMajorInput(disjoint=self.output_dim_per_node == 1, want_bits=True)
        mapped_t = soft_select_t(x, self.mapping.W, self.mapping.tau, grad_channel=channel)
        plan = _identity_plan(self.output_size, self.n, self.output_dim_per_node, x.device)
        if self._stacked == "dwn":
            return DWNLayerFunction.apply(mapped_t, self.luts, plan, self.alpha, self.beta, None, channel)
        scales = self.gradient_scale.detach().float().repeat_interleave(self.output_dim_per_node)
        return DWNLayerFunction.apply(mapped_t, self.stable_tables(), plan, 0.0, 0.0, scales, channel)

    def get_mapping_matrix(self) -> torch.Tensor:
        with torch.no_grad():
            return torch.argmax(self.mapping.W, dim=-1).view(self.output_size, self.n)

    def update_tau(self, iteration: int):
        """tau = max(tau_start * 10^(-iteration / tau_decay_iters), tau_min)."""
        self.tau = max(self.tau_start * 10.0 ** (-iteration / self.tau_decay_iters), self.tau_min)
        self.mapping.tau = self.tau
        self.mapping._cache_valid = False

    def extra_repr(self) -> str:
        flip = f", flip_prob={self.flip_probability}" if self.flip_probability > 0 else ""
        grad = f", grad_stab={self.grad_stabilization}" if self.grad_stabilization != "none" else ""
        return (f"input_size={self.input_size}, output_size={self.output_size}, "
                f"n={self.n}, tau={self.tau}, mapping=learnable{flip}{grad}")
