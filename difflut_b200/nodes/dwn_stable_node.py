"""Gradient-stabilised DWN node: DWN lookup forward, rescaled finite-difference backward.

Public surface and arithmetic follow difflut/nodes/dwn_stable_node.py:235-381: the tables are
`sigmoid(raw_luts)` with `raw_luts ~ 0.1 * N(0,1)` of shape (output_dim, 2^input_dim); the input bit is
`x >= 0.5`, LSB-first; training returns the table value, eval returns `value >= 0.5`.  Backward
(dwn_stable_node.py:145-205): the table gradient is the address histogram of the output gradient times
`gradient_scale`, the input gradient weighs table entry k by `(+-1) / (hamming(a, k without bit i) + 1)`
times `gradient_scale`, summed over the node's outputs.  `gradient_scale` is an `nn.Parameter` that
receives no gradient (the reference reads it with `.item()`).

The arithmetic runs in the feature-major layer kernels of `csrc/dwn.cu`; the non-separable
`1/(h+1)` weighting is folded into the per-step backward transform by `dl_dwn_prepare_weighted`.
"""

from typing import Callable, Optional

import torch
import torch.nn as nn

from ..registry import register_node
from .base_node import BaseNode
from .dwn_node import _check_cuda, dwn_mapped_eval

DEFAULT_DWN_STABLE_GRADIENT_SCALE: float = 1.0
DEFAULT_DWN_STABLE_USE_CUDA: bool = True
MAX_DWN_STABLE_INPUT_DIM: int = 16
FAST_DWN_STABLE_INPUT_DIM: int = 6  # up to here the weighted transform fits the 32-value-per-slot layer kernels


class DWNStableWideFunction(torch.autograd.Function):
    """N nodes with more than 6 inputs on mapped inputs xm (B, N, n), tables (N, O, 2^n) -> (B, N, O).

    Forward: table look-up (`dl_dwn_mapped_fwd`).  Backward: the reference's per-sample sums
    (dwn_stable_node.py:145-205) as `dl_dwn_stable_mapped_bwd_input` and the address histogram of the
    output gradient times `gradient_scale`."""

    @staticmethod
    def forward(ctx, xm, tables, scale):
        from .. import _native

        xm = xm.contiguous().float()
        tables = tables.contiguous().float()
        B, N, n = xm.shape
        O = tables.shape[1]
        out = torch.empty(B, N, O, device=xm.device, dtype=torch.float32)
        with torch.cuda.device(xm.device):
            _native.call("dl_dwn_mapped_fwd", xm, tables, out, B, N, n, O, 0)
        ctx.save_for_backward(xm, tables)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, g):
        from .. import _native

        xm, tables = ctx.saved_tensors
        B, N, n = xm.shape
        O = tables.shape[1]
        g = g.contiguous().float()
        scale = ctx.scale
        per_node = scale.detach().float().reshape(N).contiguous() if isinstance(scale, torch.Tensor) else None
        gxm = gt = None
        with torch.cuda.device(xm.device):
            if ctx.needs_input_grad[0]:
                gxm = torch.empty_like(xm)
                _native.call("dl_dwn_stable_mapped_bwd_input", xm, tables, g, per_node,
                             1.0 if per_node is not None else float(scale), gxm, B, N, n, O)
            if ctx.needs_input_grad[1]:
                gt = torch.empty_like(tables)
                _native.call("dl_dwn_mapped_bwd", xm, g, None, None, gt, B, N, n, O)
                gt = gt * (per_node.reshape(N, 1, 1) if per_node is not None else float(scale))
        return gxm, gt, None


def dwn_stable_mapped_forward(xm, tables, gradient_scale):
    """Training forward of N nodes on mapped inputs xm (B, N, n), tables (N, O, 2^n) -> (B, N, O).

    `gradient_scale` is a float or a tensor with one value per node.  Up to 6 inputs per node the
    feature-major layer kernels run under the identity connection map (node j reads columns
    j*n .. j*n+n-1); wider nodes take the per-sample kernels of `DWNStableWideFunction`."""
    from ..layers.fused_ops import DWNLayerFunction
    from .dwn_node import _identity_plan

    _check_cuda(xm, tables)
    B, N, n = xm.shape
    O = tables.shape[1]
    if n > MAX_DWN_STABLE_INPUT_DIM:
        raise ValueError(f"DWNStableNode supports input_dim <= {MAX_DWN_STABLE_INPUT_DIM}, got {n}")
    if n > FAST_DWN_STABLE_INPUT_DIM:
        return DWNStableWideFunction.apply(xm, tables, gradient_scale)
    if isinstance(gradient_scale, torch.Tensor):
        gradient_scale = gradient_scale.detach().float().reshape(N).repeat_interleave(O)
    plan = _identity_plan(N, n, O, xm.device)
    out = DWNLayerFunction.apply(xm.reshape(B, N * n), tables, plan, 0.0, 0.0, gradient_scale)
    return out.reshape(B, N, O)


@register_node("dwn_stable")
class DWNStableNode(BaseNode):
    """DWN node with sigmoid-parameterised tables and a `1/(hamming+1)`-weighted, rescaled backward."""

    def __init__(
        self,
        input_dim: Optional[int] = None,
        output_dim: Optional[int] = None,
        use_cuda: bool = True,
        regularizers: Optional[dict] = None,
        gradient_scale: float = 1.25,
        init_fn: Optional[Callable] = None,
        init_kwargs: Optional[dict] = None,
    ):
        super().__init__(input_dim=input_dim, output_dim=output_dim, regularizers=regularizers,
                         init_fn=init_fn, init_kwargs=init_kwargs)
        if self.num_inputs > MAX_DWN_STABLE_INPUT_DIM:
            raise ValueError(
                f"DWNStableNode supports input_dim <= {MAX_DWN_STABLE_INPUT_DIM}, got {self.num_inputs}"
            )
        self.use_cuda = bool(use_cuda)  # accepted for compatibility; there is one (CUDA) path
        self.gradient_scale = nn.Parameter(torch.tensor(gradient_scale))
        self.raw_luts = nn.Parameter(torch.randn(self.num_outputs, 2 ** self.num_inputs) * 0.1)
        self._apply_init_fn(self.raw_luts, name="raw_luts")

    @classmethod
    def _view_of(cls, layer, index: int) -> "DWNStableNode":
        """Node object whose parameters are row `index` of a layer's stacked parameters (no own storage)."""
        node = cls.__new__(cls)
        nn.Module.__init__(node)
        node.input_dim, node.output_dim = layer.n, layer.output_dim_per_node
        node.regularizers = layer._node_regularizers
        node.init_fn, node.init_kwargs = layer._node_init_fn, layer._node_init_kwargs
        node.use_cuda = True
        node.raw_luts = layer.raw_luts[index]  # views: in-place edits and gradients reach the layer
        node.gradient_scale = layer.gradient_scale[index]
        node.training = layer.training
        return node

    def _get_luts(self) -> torch.Tensor:
        return torch.sigmoid(self.raw_luts)

    def _validate(self, x: torch.Tensor) -> None:
        if x.dim() != 2 or x.shape[1] != self.num_inputs:
            raise ValueError(f"DWNStableNode expects (batch, {self.num_inputs}) input, got {tuple(x.shape)}")

    def forward_train(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        scale = float(self.gradient_scale.detach())
        return dwn_stable_mapped_forward(x.unsqueeze(1), self._get_luts().unsqueeze(0), scale).squeeze(1)

    def forward_eval(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        return dwn_mapped_eval(x.unsqueeze(1), self._get_luts().unsqueeze(0)).squeeze(1)

    def _builtin_regularization(self) -> torch.Tensor:
        return torch.tensor(0.0, device=self.raw_luts.device, requires_grad=False)
