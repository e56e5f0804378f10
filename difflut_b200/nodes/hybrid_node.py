"""Hybrid node: DWN look-up forward, probabilistic backward.

Public surface and arithmetic follow difflut/nodes/hybrid_node.py:245-378: tables are
`sigmoid(raw_luts)` with `raw_luts ~ 0.1 * N(0,1)` of shape (output_dim, 2^input_dim); the forward
addresses the table with bits `x >= 0.5` (LSB-first), eval returns `value >= 0.5`.  Backward
(hybrid_node.py:173-224) uses the multilinear weights P_a(x) = prod_i (a_i ? x_i : 1 - x_i) of the
real-valued input: table gradient `sum_b g * P_a`, input gradient
`sum_a P_a * (a_i - x_i) / (x_i (1 - x_i) + 1e-8) * table[a]`, i.e. the product-rule derivative times
`x(1-x) / (x(1-x) + 1e-8)` (zero at exactly binary inputs).

The arithmetic runs in `csrc/dwn.cu` (forward) and `csrc/prob.cu` (`dl_hybrid_bwd_t`).
"""

from typing import Callable, Optional

import torch
import torch.nn as nn

from ..registry import register_node
from .base_node import BaseNode
from .dwn_node import _check_cuda, dwn_mapped_eval

DEFAULT_HYBRID_USE_CUDA: bool = True
MAX_HYBRID_INPUT_DIM: int = 16
FAST_HYBRID_INPUT_DIM: int = 6  # up to here the layer kernel keeps a node's 2^n table gradient in registers


class HybridWideFunction(torch.autograd.Function):
    """N hybrid nodes with more than 6 inputs on mapped inputs xm (B, N, n), tables (N, O, 2^n) -> (B, N, O).

    Forward: table look-up (`dl_dwn_mapped_fwd`); backward: the probabilistic gradient of
    hybrid_node.py:160-224 as `dl_hybrid_mapped_bwd`."""

    @staticmethod
    def forward(ctx, xm, tables):
        from .. import _native

        xm = xm.contiguous().float()
        tables = tables.contiguous().float()
        B, N, n = xm.shape
        O = tables.shape[1]
        out = torch.empty(B, N, O, device=xm.device, dtype=torch.float32)
        with torch.cuda.device(xm.device):
            _native.call("dl_dwn_mapped_fwd", xm, tables, out, B, N, n, O, 0)
        ctx.save_for_backward(xm, tables)
        return out

    @staticmethod
    def backward(ctx, g):
        from .. import _native

        xm, tables = ctx.saved_tensors
        B, N, n = xm.shape
        O = tables.shape[1]
        g = g.contiguous().float()
        gxm = torch.empty_like(xm) if ctx.needs_input_grad[0] else None
        gt = torch.empty_like(tables) if ctx.needs_input_grad[1] else None
        if gxm is not None or gt is not None:
            with torch.cuda.device(xm.device):
                _native.call("dl_hybrid_mapped_bwd", xm, tables, g, gxm, gt, B, N, n, O)
        return gxm, gt


def hybrid_mapped_forward(xm, tables):
    """Training forward of N nodes on mapped inputs xm (B, N, n), tables (N, O, 2^n) -> (B, N, O)."""
    from ..layers.fused_ops import HybridLayerFunction
    from .dwn_node import _identity_plan

    _check_cuda(xm, tables)
    B, N, n = xm.shape
    O = tables.shape[1]
    if n > MAX_HYBRID_INPUT_DIM:
        raise ValueError(f"HybridNode supports input_dim <= {MAX_HYBRID_INPUT_DIM}, got {n}")
    if n > FAST_HYBRID_INPUT_DIM:
        return HybridWideFunction.apply(xm, tables)
    plan = _identity_plan(N, n, O, xm.device)
    return HybridLayerFunction.apply(xm.reshape(B, N * n), tables, plan).reshape(B, N, O)


@register_node("hybrid")
class HybridNode(BaseNode):
    """Discrete DWN forward with the smooth probabilistic gradient."""

    def __init__(
        self,
        input_dim: Optional[int] = None,
        output_dim: Optional[int] = None,
        use_cuda: bool = True,
        regularizers: Optional[dict] = None,
        init_fn: Optional[Callable] = None,
        init_kwargs: Optional[dict] = None,
    ):
        super().__init__(input_dim=input_dim, output_dim=output_dim, regularizers=regularizers,
                         init_fn=init_fn, init_kwargs=init_kwargs)
        if self.num_inputs > MAX_HYBRID_INPUT_DIM:
            raise ValueError(f"HybridNode supports input_dim <= {MAX_HYBRID_INPUT_DIM}, got {self.num_inputs}")
        self.use_cuda = bool(use_cuda)  # accepted for compatibility; there is one (CUDA) path
        self.raw_luts = nn.Parameter(torch.randn(self.num_outputs, 2 ** self.num_inputs) * 0.1)
        self._apply_init_fn(self.raw_luts, name="raw_luts")
        self.register_buffer("binary_combinations", self.binary_patterns(self.num_inputs, "cpu"))

    @staticmethod
    def binary_patterns(n: int, device) -> torch.Tensor:
        """(2^n, n) LSB-first patterns, the reference's `binary_combinations` buffer."""
        a = torch.arange(2 ** n, device=device)
        return ((a[:, None] >> torch.arange(n, device=device)[None, :]) & 1).float()

    @classmethod
    def _view_of(cls, layer, index: int) -> "HybridNode":
        """Node object whose `raw_luts` is row `index` of a layer's stacked parameter (no own storage)."""
        node = cls.__new__(cls)
        nn.Module.__init__(node)
        node.input_dim, node.output_dim = layer.n, layer.output_dim_per_node
        node.regularizers = layer._node_regularizers
        node.init_fn, node.init_kwargs = layer._node_init_fn, layer._node_init_kwargs
        node.use_cuda = True
        node.raw_luts = layer.raw_luts[index]  # a view: in-place edits and gradients reach the layer
        node.register_buffer("binary_combinations", cls.binary_patterns(layer.n, layer.raw_luts.device))
        node.training = layer.training
        return node

    def _get_luts(self) -> torch.Tensor:
        return torch.sigmoid(self.raw_luts)

    def _validate(self, x: torch.Tensor) -> None:
        if x.dim() != 2 or x.shape[1] != self.num_inputs:
            raise ValueError(f"HybridNode expects (batch, {self.num_inputs}) input, got {tuple(x.shape)}")

    def forward_train(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        return hybrid_mapped_forward(x.unsqueeze(1), self._get_luts().unsqueeze(0)).squeeze(1)

    def forward_eval(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        return dwn_mapped_eval(x.unsqueeze(1), self._get_luts().unsqueeze(0)).squeeze(1)

    def _builtin_regularization(self) -> torch.Tensor:
        return torch.tensor(0.0, device=self.raw_luts.device, requires_grad=False)
