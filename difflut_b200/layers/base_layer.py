"""Base LUT layer: stacked node parameters behind the reference's per-node interface.

The reference layer owns `nn.ModuleList([node_type(...) for _ in range(N)])` and loops over
it (difflut/layers/base_layer.py:342-576).  Here, when `node_type` is one of the package's
own DWN / DWNStable / Hybrid / Probabilistic nodes, the layer owns ONE stacked parameter (`luts (N, O, 2^n)`,
`raw_luts (N, O, 2^n)` (+ `gradient_scale (N,)` for DWNStable), or `raw_weights (N, 2^n, O)`) and runs one kernel
per pass; `layer.nodes` is a lazy sequence of node views so that `layer.nodes[i].luts`, `len(layer.nodes)`, per-node calls, initializers and
regularizers keep working, and the state dict is written with the reference's per-node keys
(`nodes.{i}.luts` ...).  Any other node class keeps the reference structure (a ModuleList,
the gather kernel and a per-node loop), which is API compatibility, not a second backend.
"""

import warnings
from abc import ABC, abstractmethod
from typing import Optional, Type

import torch
import torch.nn as nn

from ..nodes.base_node import validate_node_dims, validate_regularizers
from ..nodes.dwn_node import DWNNode, MAX_DWN_INPUT_DIM, default_alpha, default_beta
from ..nodes.dwn_stable_node import DWNStableNode, MAX_DWN_STABLE_INPUT_DIM
from ..nodes.hybrid_node import HybridNode, MAX_HYBRID_INPUT_DIM
from ..nodes.node_config import NodeConfig
from ..nodes.probabilistic_node import ProbabilisticNode
from ..utils.warnings import warn_default_value
from .fused_ops import ConnectionPlan
from .layer_config import LayerConfig, check_flip_probability, check_grad_mode, check_positive

DEFAULT_LAYER_FLIP_PROBABILITY: float = 0.0
DEFAULT_LAYER_GRAD_STABILIZATION: str = "none"
DEFAULT_LAYER_GRAD_TARGET_STD: float = 1.0
DEFAULT_LAYER_GRAD_SUBTRACT_MEAN: bool = False
DEFAULT_LAYER_GRAD_EPSILON: float = 1e-8
LAYER_REUSE_WARNING_THRESHOLD: int = 10
LAYER_UNDERUSE_WARNING_DIVISOR: int = 10
LAYER_MAX_NODE_INPUT_DIM: int = 15


class LUTLayerMixin(nn.Module):
    """Bit-flip augmentation and gradient rescaling options shared by LUT layers.

    As in the reference, RandomLayer / LearnableLayer override `forward` and never call these
    (difflut/layers/random_layer.py:306-340), so they are host-side torch code, not kernels.
    """

    def _init_lut_layer_mixin(self, layer_config=None, flip_probability=None, grad_stabilization=None,
                              grad_target_std=None, grad_subtract_mean=None, grad_epsilon=None) -> None:
        if layer_config is not None:
            if not isinstance(layer_config, LayerConfig):
                raise TypeError(
                    f"layer_config must be a LayerConfig instance, got {type(layer_config)}. "
                    f"Use: layer_config=LayerConfig(flip_probability=0.1, ...)"
                )
            self.flip_probability = layer_config.flip_probability
            self.grad_stabilization = layer_config.grad_stabilization
            self.grad_target_std = layer_config.grad_target_std
            self.grad_subtract_mean = layer_config.grad_subtract_mean
            self.grad_epsilon = layer_config.grad_epsilon
        else:
            def pick(value, default, name):
                if value is None:
                    warn_default_value(name, default, stacklevel=4)
                    return default
                return value

            self.flip_probability = pick(flip_probability, DEFAULT_LAYER_FLIP_PROBABILITY, "flip_probability")
            check_flip_probability(self.flip_probability)
            self.grad_stabilization = pick(grad_stabilization, DEFAULT_LAYER_GRAD_STABILIZATION, "grad_stabilization")
            check_grad_mode(self.grad_stabilization)
            self.grad_target_std = pick(grad_target_std, DEFAULT_LAYER_GRAD_TARGET_STD, "grad_target_std")
            check_positive("grad_target_std", self.grad_target_std, "Example: grad_target_std=1.0 for unit variance")
            self.grad_subtract_mean = pick(grad_subtract_mean, DEFAULT_LAYER_GRAD_SUBTRACT_MEAN, "grad_subtract_mean")
            self.grad_epsilon = pick(grad_epsilon, DEFAULT_LAYER_GRAD_EPSILON, "grad_epsilon")
            check_positive("grad_epsilon", self.grad_epsilon, "Used for numerical stability in variance calculation")
        self._flip_mask_buffer = None

    @staticmethod
    def _draw_seed() -> int:
        """A fresh 62-bit seed from torch's CPU generator (reproducible under torch.manual_seed)."""
        return int(torch.randint(0, 2 ** 62, (1,), dtype=torch.int64).item())

    def _apply_bit_flip(self, x: torch.Tensor) -> torch.Tensor:
        """x -> 1-x on a random `flip_probability` fraction; the flip carries no gradient.

        As in the reference (base_layer.py:189-262): below a probability of 0.05 exactly
        int(numel * p) distinct positions flip, the first entries of `torch.randperm(numel)` on the tensor's
        device (`dl_flip_at`); from 0.05 on every element flips independently (`dl_flip_rows`)."""
        if self.flip_probability <= 0.0 or not self.training:
            return x
        if x.is_cuda:
            if self.flip_probability < 0.05:
                positions = self._draw_flip_positions(x.numel(), x.device)
                return x if positions is None else _FlipAtFunction.apply(x, positions)
            return _FlipFunction.apply(x, float(self.flip_probability), self._draw_seed())
        if self.flip_probability < 0.05:
            count = int(x.numel() * self.flip_probability)
            if count == 0:
                return x
            mask = torch.zeros(x.numel(), dtype=torch.bool, device=x.device)
            mask[torch.randperm(x.numel(), device=x.device)[:count]] = True
            mask = mask.view_as(x)
        else:
            mask = torch.bernoulli(torch.full(x.shape, float(self.flip_probability), device=x.device)).bool()
        delta = torch.where(mask, 1.0 - 2.0 * x.detach(), torch.zeros_like(x))
        return x + delta

    def _draw_flip_positions(self, numel: int, device) -> Optional[torch.Tensor]:
        """The positions the reference's sparse rule flips (base_layer.py:242-254), or None when there are none."""
        count = int(numel * self.flip_probability)
        if count == 0:
            return None
        return torch.randperm(numel, device=device)[:count].contiguous()

    def _apply_gradient_stabilization(self, grad: torch.Tensor) -> torch.Tensor:
        """(g - mean) * sqrt(target_std / (mean(g^2) + eps)), over the layer or per sample
        (`dl_grad_rescale` for CUDA tensors)."""
        if self.grad_stabilization == "none" or not self.training or grad is None:
            return grad
        if grad.is_cuda and grad.dim() == 2:
            from .. import _native

            g = grad.contiguous().float()
            out = torch.empty_like(g)
            per_row = 0 if self.grad_stabilization == "layerwise" else 1
            with torch.cuda.device(g.device):
                scratch = None
                if not per_row:
                    scratch = torch.empty(int(_native.lib().dl_grad_rescale_scratch_doubles()), device=g.device,
                                          dtype=torch.float64)
                _native.call("dl_grad_rescale", g, out, g.shape[0], g.shape[1], per_row, float(self.grad_target_std),
                             1 if self.grad_subtract_mean else 0, float(self.grad_epsilon), scratch)
            return out
        dims = None if self.grad_stabilization == "layerwise" else 1
        g = grad.clone()
        if self.grad_subtract_mean:
            g = g - (g.mean() if dims is None else g.mean(dim=1, keepdim=True))
        var = g.pow(2).mean() if dims is None else g.pow(2).mean(dim=1, keepdim=True)
        return g * torch.sqrt(torch.tensor(self.grad_target_std, device=grad.device) / (var + self.grad_epsilon))


class _FlipFunction(torch.autograd.Function):
    """out = 1 - x on a Bernoulli(p) subset, identity gradient (the reference adds a detached delta)."""

    @staticmethod
    def forward(ctx, x, probability, seed):
        from .. import _native

        x = x.contiguous().float()
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _native.call("dl_flip_rows", x, out, x.numel(), probability, seed)
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class _FlipAtFunction(torch.autograd.Function):
    """out = 1 - x at the given positions, identity gradient (the reference adds a detached delta)."""

    @staticmethod
    def forward(ctx, x, positions):
        from .. import _native

        x = x.contiguous().float()
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _native.call("dl_flip_at", x, out, positions, x.numel(), positions.numel())
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None


class _NodeViews:
    """`layer.nodes` for a stacked layer: len / index / iterate; items are built on access so a
    view always refers to the layer's current parameter storage."""

    def __init__(self, layer):
        object.__setattr__(self, "_layer", layer)

    def __len__(self) -> int:
        return self._layer.output_size

    def __getitem__(self, i):
        N = len(self)
        if isinstance(i, slice):
            return [self[k] for k in range(*i.indices(N))]
        if i < 0:
            i += N
        if not 0 <= i < N:
            raise IndexError(f"node index {i} out of range for {N} nodes")
        return self._layer._node_class._view_of(self._layer, i)

    def __iter__(self):
        for i in range(len(self)):
            yield self[i]


class BaseLUTLayer(ABC, LUTLayerMixin, nn.Module):
    """(B, input_size) -> (B, output_size * output_dim_per_node)."""

    def __init__(
        self,
        input_size: int,
        output_size: int,
        node_type: Type[nn.Module],
        node_kwargs: NodeConfig,
        layer_config: Optional[LayerConfig] = None,
        flip_probability: Optional[float] = None,
        grad_stabilization: Optional[str] = None,
        grad_target_std: Optional[float] = None,
        grad_subtract_mean: Optional[bool] = None,
        grad_epsilon: Optional[float] = None,
    ) -> None:
        super().__init__()
        if not isinstance(input_size, int) or input_size <= 0:
            raise ValueError(
                f"input_size must be a positive integer, got {input_size}. "
                f"This typically comes from an encoder output or previous layer output."
            )
        if not isinstance(output_size, int) or output_size <= 0:
            raise ValueError(
                f"output_size must be a positive integer, got {output_size}. "
                f"This is the number of nodes in the layer."
            )
        self._init_lut_layer_mixin(layer_config, flip_probability, grad_stabilization, grad_target_std,
                                   grad_subtract_mean, grad_epsilon)
        self.input_size = input_size
        self.output_size = output_size
        self._plan_cache = None
        kwargs = node_kwargs.to_dict() if isinstance(node_kwargs, NodeConfig) else dict(node_kwargs or {})
        self._node_class = node_type
        if node_type is DWNNode:
            self._stacked = "dwn"
            self._init_stacked_dwn(**kwargs)
        elif node_type is DWNStableNode:
            self._stacked = "dwn_stable"
            self._init_stacked_dwn_stable(**kwargs)
        elif node_type is HybridNode:
            self._stacked = "hybrid"
            self._init_stacked_hybrid(**kwargs)
        elif node_type is ProbabilisticNode:
            self._stacked = "probabilistic"
            self._init_stacked_prob(**kwargs)
        else:
            self._stacked = None
            self.nodes = nn.ModuleList([node_type(**kwargs) for _ in range(output_size)])
            self.n = self.nodes[0].num_inputs
            self.output_dim_per_node = self.nodes[0].num_outputs
        self._validate_layer_config()

    # ------------------------------------------------------------------ stacked construction
    def _common_node_args(self, input_dim, output_dim, regularizers, init_fn, init_kwargs):
        self.n, self.output_dim_per_node = validate_node_dims(input_dim, output_dim, stacklevel=5)
        self._node_regularizers = validate_regularizers(regularizers or {})
        if init_fn is not None and not callable(init_fn):
            raise TypeError(f"init_fn must be callable, but got {type(init_fn).__name__}.")
        self._node_init_fn = init_fn
        self._node_init_kwargs = dict(init_kwargs or {})
        if not isinstance(self._node_init_kwargs, dict):
            raise TypeError("init_kwargs must be a dict")

    def _init_rows(self, param: torch.Tensor, name: str) -> None:
        """Apply the node initializer row by row, each row shaped like the reference's node parameter."""
        if self._node_init_fn is None:
            return
        with torch.no_grad():
            for i in range(param.shape[0]):
                try:
                    self._node_init_fn(param[i], **self._node_init_kwargs)
                except Exception as e:
                    raise RuntimeError(
                        f"Initialization of '{name}' failed with error: {e}. "
                        f"Check that init_fn is compatible with the parameter and init_kwargs are correct."
                    )

    def _init_stacked_dwn(self, input_dim=None, output_dim=None, use_cuda=True, regularizers=None, alpha=None,
                          beta=None, clamp_luts=True, init_fn=None, init_kwargs=None):
        init_kwargs = dict(init_kwargs or {})
        if "input_dim" not in init_kwargs and input_dim is not None:
            init_kwargs["input_dim"] = input_dim
        self._common_node_args(input_dim, output_dim, regularizers, init_fn, init_kwargs)
        if self.n > MAX_DWN_INPUT_DIM:
            raise ValueError(f"DWNNode supports input_dim <= {MAX_DWN_INPUT_DIM}, got {self.n}")
        if alpha is None:
            alpha = default_alpha(self.n)
            warn_default_value("alpha", alpha, stacklevel=4)
        if beta is None:
            beta = default_beta()
            warn_default_value("beta", beta, stacklevel=4)
        self.alpha, self.beta = float(alpha), float(beta)
        self.luts = nn.Parameter(torch.rand(self.output_size, self.output_dim_per_node, 2 ** self.n))
        self._init_rows(self.luts.data, "luts")
        self.nodes = _NodeViews(self)

    def _init_stacked_dwn_stable(self, input_dim=None, output_dim=None, use_cuda=True, regularizers=None,
                                 gradient_scale=1.25, init_fn=None, init_kwargs=None):
        self._common_node_args(input_dim, output_dim, regularizers, init_fn, init_kwargs)
        if self.n > MAX_DWN_STABLE_INPUT_DIM:
            raise ValueError(f"DWNStableNode supports input_dim <= {MAX_DWN_STABLE_INPUT_DIM}, got {self.n}")
        self.gradient_scale = nn.Parameter(torch.full((self.output_size,), float(gradient_scale)))
        self.raw_luts = nn.Parameter(torch.randn(self.output_size, self.output_dim_per_node, 2 ** self.n) * 0.1)
        self._init_rows(self.raw_luts.data, "raw_luts")
        self.nodes = _NodeViews(self)

    def _init_stacked_hybrid(self, input_dim=None, output_dim=None, use_cuda=True, regularizers=None, init_fn=None,
                             init_kwargs=None):
        self._common_node_args(input_dim, output_dim, regularizers, init_fn, init_kwargs)
        if self.n > MAX_HYBRID_INPUT_DIM:
            raise ValueError(f"HybridNode supports input_dim <= {MAX_HYBRID_INPUT_DIM}, got {self.n}")
        self.raw_luts = nn.Parameter(torch.randn(self.output_size, self.output_dim_per_node, 2 ** self.n) * 0.1)
        self._init_rows(self.raw_luts.data, "raw_luts")
        self.nodes = _NodeViews(self)

    def stable_tables(self) -> torch.Tensor:
        """sigmoid(raw_luts) (N, O, 2^n) of a DWNStable / Hybrid layer (dwn_stable_node.py:310-316,
        hybrid_node.py:308-314)."""
        return torch.sigmoid(self.raw_luts)

    def _init_stacked_prob(self, input_dim=None, output_dim=None, init_fn=None, init_kwargs=None,
                           regularizers=None, temperature=1.0, eval_mode="expectation", use_cuda=True):
        self._common_node_args(input_dim, output_dim, regularizers, init_fn, init_kwargs)
        assert eval_mode in {"expectation", "deterministic", "threshold"}, "Invalid eval_mode"
        self.eval_mode = eval_mode
        self.temperature = float(temperature)
        self.raw_weights = nn.Parameter(torch.randn(self.output_size, 2 ** self.n, self.output_dim_per_node))
        self._init_rows(self.raw_weights.data, "raw_weights")
        self.nodes = _NodeViews(self)

    # ------------------------------------------------------------------ reference-format state dict
    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        if self._stacked is None:
            return
        if self._stacked == "dwn":
            stacked = destination.pop(prefix + "luts")
            dev = stacked.device
            for i in range(self.output_size):
                destination[f"{prefix}nodes.{i}.alpha"] = torch.tensor(self.alpha, dtype=torch.float32, device=dev)
                destination[f"{prefix}nodes.{i}.beta"] = torch.tensor(self.beta, dtype=torch.float32, device=dev)
                destination[f"{prefix}nodes.{i}.luts"] = stacked[i]
        elif self._stacked == "dwn_stable":
            stacked = destination.pop(prefix + "raw_luts")
            scales = destination.pop(prefix + "gradient_scale")
            for i in range(self.output_size):
                destination[f"{prefix}nodes.{i}.gradient_scale"] = scales[i]
                destination[f"{prefix}nodes.{i}.raw_luts"] = stacked[i]
        elif self._stacked == "hybrid":
            stacked = destination.pop(prefix + "raw_luts")
            patterns = HybridNode.binary_patterns(self.n, stacked.device)
            for i in range(self.output_size):
                destination[f"{prefix}nodes.{i}.raw_luts"] = stacked[i]
                destination[f"{prefix}nodes.{i}.binary_combinations"] = patterns
        else:
            stacked = destination.pop(prefix + "raw_weights")
            dev = stacked.device
            patterns = ProbabilisticNode.binary_patterns(self.n, dev)
            for i in range(self.output_size):
                destination[f"{prefix}nodes.{i}.raw_weights"] = stacked[i]
                destination[f"{prefix}nodes.{i}.temperature"] = torch.tensor(self.temperature, device=dev)
                destination[f"{prefix}nodes.{i}.binary_combinations"] = patterns

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                              error_msgs):
        if self._stacked is not None:
            name = {"dwn": "luts", "dwn_stable": "raw_luts", "hybrid": "raw_luts",
                    "probabilistic": "raw_weights"}[self._stacked]
            first = f"{prefix}nodes.0.{name}"
            if first in state_dict and (prefix + name) not in state_dict:
                rows = []
                for i in range(self.output_size):
                    key = f"{prefix}nodes.{i}.{name}"
                    if key not in state_dict:
                        missing_keys.append(key)
                        rows = None
                        break
                    rows.append(state_dict[key])
                if rows is not None:
                    state_dict[prefix + name] = torch.stack([r.detach() for r in rows])
                if self._stacked == "dwn_stable" and f"{prefix}nodes.0.gradient_scale" in state_dict:
                    state_dict[prefix + "gradient_scale"] = torch.stack(
                        [state_dict[f"{prefix}nodes.{i}.gradient_scale"].detach().reshape(())
                         for i in range(self.output_size)])
                if self._stacked == "dwn" and f"{prefix}nodes.0.alpha" in state_dict:
                    self.alpha = float(state_dict[f"{prefix}nodes.0.alpha"])
                    self.beta = float(state_dict[f"{prefix}nodes.0.beta"])
                if self._stacked == "probabilistic" and f"{prefix}nodes.0.temperature" in state_dict:
                    self.temperature = float(state_dict[f"{prefix}nodes.0.temperature"])
            for key in [k for k in state_dict if k.startswith(prefix + "nodes.")]:
                del state_dict[key]
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                      error_msgs)

    # ------------------------------------------------------------------ checks
    def _validate_layer_config(self) -> None:
        total = self.output_size * self.n
        if total > self.input_size * LAYER_REUSE_WARNING_THRESHOLD:
            warnings.warn(
                f"BaseLUTLayer: Creating {total} node input connections from only {self.input_size} input "
                f"features. Each input feature will be reused {total // self.input_size}x on average. "
                f"This may lead to overfitting.",
                UserWarning,
                stacklevel=2,
            )
        if total < self.input_size // LAYER_UNDERUSE_WARNING_DIVISOR:
            warnings.warn(
                f"BaseLUTLayer: Creating only {total} node inputs from {self.input_size} input features. "
                f"Most input features will be unused.",
                UserWarning,
                stacklevel=2,
            )
        if self.n > LAYER_MAX_NODE_INPUT_DIM:
            warnings.warn(
                f"BaseLUTLayer: Node input dimension (n={self.n}) is quite large. "
                f"LUT nodes with >15 inputs need 2^{self.n} entries each.",
                UserWarning,
                stacklevel=2,
            )

    def _validate_input_dims(self, x: torch.Tensor) -> None:
        if x.dim() != 2:
            raise ValueError(
                f"BaseLUTLayer expects 2D input (batch_size, input_size), "
                f"but got shape {x.shape} with {x.dim()} dimensions."
            )
        batch_size, feat = x.shape
        if feat != self.input_size:
            raise ValueError(
                f"BaseLUTLayer expected input with {self.input_size} features, "
                f"but got {feat} features. Shape: {x.shape}."
            )
        if batch_size == 0:
            raise ValueError(f"BaseLUTLayer requires non-empty batch, got batch_size={batch_size}")
        if not x.is_cuda:
            raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")

    # ------------------------------------------------------------------ mapping plumbing
    def _plan_for(self, indices: torch.Tensor, device: torch.device, tag) -> ConnectionPlan:
        """ConnectionPlan for `indices`, cached until the indices object, device or tag changes."""
        key = (tag, str(device), indices.data_ptr(), indices._version)
        if self._plan_cache is None or self._plan_cache[0] != key:
            plan = ConnectionPlan(indices, self.input_size, self.output_dim_per_node, device)
            self._plan_cache = (key, plan)
        return self._plan_cache[1]

    @abstractmethod
    def get_mapping(self, x: torch.Tensor) -> torch.Tensor:
        """(B, input_size) -> (B, output_size, n) mapped node inputs."""

    def get_mapping_indices(self):
        return None

    def _own_params(self):
        """The stacked parameter tensors the node arithmetic of this layer reads, as a tuple."""
        if self._stacked == "dwn":
            return (self.luts,)
        if self._stacked == "dwn_stable":
            return (self.raw_luts, self.gradient_scale)
        if self._stacked == "hybrid":
            return (self.raw_luts,)
        if self._stacked == "probabilistic":
            return (self.raw_weights,)
        return ()

    def _apply_plan(self, x: torch.Tensor, plan: ConnectionPlan, params=None, geom=None) -> torch.Tensor:
        """Layer arithmetic (B, I) -> (B, N*O) under connection plan `plan` with parameters `params`
        (default: this layer's own).  Other callers pass the concatenated parameters of several layers
        of the same configuration together with their combined plan, which runs them as one layer.
        With `geom` (a PatchGeometry) x is an image batch and the samples are its patches; node types
        that only look at `x >= 0.5` then never materialise the patches."""
        from .fused_ops import (DWNLayerFunction, GatherFunction, HybridLayerFunction, PatchFunction,
                                ProbLayerFunction, dwn_levels_eval)

        params = self._own_params() if params is None else params
        kind, fast = self._stacked, self.n <= 6
        if kind == "dwn" and fast:
            if self.training:
                return DWNLayerFunction.apply(x, params[0], plan, self.alpha, self.beta, None, geom)
            return dwn_levels_eval(x, [(params[0], plan)], geom)
        if kind == "dwn_stable" and fast:
            tables = torch.sigmoid(params[0])
            if self.training:
                scales = params[1].detach().float().repeat_interleave(self.output_dim_per_node)
                return DWNLayerFunction.apply(x, tables, plan, 0.0, 0.0, scales, geom)
            return dwn_levels_eval(x, [(tables, plan)], geom)
        if kind == "hybrid" and fast and not self.training:
            return dwn_levels_eval(x, [(torch.sigmoid(params[0]), plan)], geom)
        if geom is not None:
            x = PatchFunction.apply(x, geom)
        if kind == "hybrid" and fast:
            return HybridLayerFunction.apply(x, torch.sigmoid(params[0]), plan)
        if kind == "probabilistic" and fast and self.training:
            return ProbLayerFunction.apply(x, params[0], plan, self.temperature, None, 1.0)
        return self._run_nodes(GatherFunction.apply(x, plan), params)

    def _run_nodes(self, mapped: torch.Tensor, params=None) -> torch.Tensor:
        """Node arithmetic on materialised inputs (B, N, n) -> (B, N*O)."""
        B = mapped.shape[0]
        params = self._own_params() if params is None else params
        if self._stacked == "dwn":
            from ..nodes.dwn_node import dwn_mapped_eval, dwn_mapped_forward

            out = (dwn_mapped_forward(mapped, params[0], self.alpha, self.beta) if self.training
                   else dwn_mapped_eval(mapped, params[0]))
            return out.reshape(B, -1)
        if self._stacked == "dwn_stable":
            from ..nodes.dwn_node import dwn_mapped_eval
            from ..nodes.dwn_stable_node import dwn_stable_mapped_forward

            tables = torch.sigmoid(params[0])
            out = (dwn_stable_mapped_forward(mapped, tables, params[1]) if self.training
                   else dwn_mapped_eval(mapped, tables))
            return out.reshape(B, -1)
        if self._stacked == "hybrid":
            from ..nodes.dwn_node import dwn_mapped_eval
            from ..nodes.hybrid_node import hybrid_mapped_forward

            tables = torch.sigmoid(params[0])
            out = hybrid_mapped_forward(mapped, tables) if self.training else dwn_mapped_eval(mapped, tables)
            return out.reshape(B, -1)
        if self._stacked == "probabilistic":
            from ..nodes.probabilistic_node import prob_mapped_eval, prob_mapped_forward

            out = (prob_mapped_forward(mapped, params[0], self.temperature) if self.training
                   else prob_mapped_eval(mapped, params[0], self.temperature))
            return out.reshape(B, -1)
        outs = [node(mapped[:, i, :]) for i, node in enumerate(self.nodes)]
        return torch.stack(outs, dim=1).reshape(B, -1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Generic path with the mixin features (what difflut/layers/base_layer.py:508-564 does)."""
        self._validate_input_dims(x)
        if self.training and self.flip_probability > 0.0:
            x = self._apply_bit_flip(x)
        out = self._run_nodes(self.get_mapping(x))
        if self.grad_stabilization != "none" and self.training and out.requires_grad:
            out.register_hook(self._apply_gradient_stabilization)
        return out

    def regularization(self) -> torch.Tensor:
        params = list(self.parameters())
        total = torch.tensor(0.0, device=params[0].device if params else "cpu")
        if self._stacked is not None and not self._node_regularizers:
            return total  # the built-in term of DWN / Probabilistic nodes is zero
        for node in self.nodes:
            if hasattr(node, "regularization") and callable(node.regularization):
                total = total + node.regularization()
        return total
