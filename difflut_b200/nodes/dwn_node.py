"""DWN node: hard LUT lookup forward, extended-finite-difference (EFD) backward.

Public surface and arithmetic follow difflut/nodes/dwn_node.py:341-544:
input bit = `x >= 0.5`, LSB-first address, output = raw table value in training and
`value >= 0.5` in eval; backward weights `alpha * (+-1) * beta^hamming` with defaults
alpha = 0.5*0.75^(n-1), beta = 0.25/0.75.  The arithmetic runs in the CUDA kernels of
`csrc/dwn.cu` through `dwn_mapped_forward` below (any N nodes at once; a standalone node is N=1).
"""

from typing import Callable, Optional

import torch
import torch.nn as nn

from .. import _native
from ..registry import register_node
from ..utils.warnings import warn_default_value
from .base_node import BaseNode

DWN_ALPHA_BASE: float = 0.5
DWN_ALPHA_DECAY: float = 0.75
DWN_BETA_NUMERATOR: float = 0.25
DWN_BETA_DENOMINATOR: float = 0.75
DWN_BINARY_THRESHOLD: float = 0.5
DEFAULT_DWN_USE_CUDA: bool = True
DEFAULT_DWN_CLAMP_LUTS: bool = True
MAX_DWN_INPUT_DIM: int = 16


def default_alpha(n: int) -> float:
    return DWN_ALPHA_BASE * (DWN_ALPHA_DECAY ** (n - 1))


def default_beta() -> float:
    return DWN_BETA_NUMERATOR / DWN_BETA_DENOMINATOR


def _check_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("difflut_b200 DWN kernels run on CUDA tensors only (no CPU fallback)")


class DWNMappedFunction(torch.autograd.Function):
    """N nodes on already-mapped inputs: xm (B,N,n), tables (N,O,2^n) -> (B,N,O).

    Counterpart of EFDFunction (difflut/nodes/dwn_node.py:58-128) for a whole layer.
    """

    @staticmethod
    def forward(ctx, xm, tables, alpha, beta):
        _check_cuda(xm, tables)
        xm = xm.contiguous().float()
        tables = tables.contiguous().float()
        B, N, n = xm.shape
        O = tables.shape[1]
        out = torch.empty(B, N, O, device=xm.device, dtype=torch.float32)
        with torch.cuda.device(xm.device):
            _native.call("dl_dwn_mapped_fwd", xm, tables, out, B, N, n, O, 0)
        ctx.save_for_backward(xm, tables)
        ctx.alpha, ctx.beta = float(alpha), float(beta)
        return out

    @staticmethod
    def backward(ctx, g):
        xm, tables = ctx.saved_tensors
        B, N, n = xm.shape
        O, L = tables.shape[1], tables.shape[2]
        g = g.contiguous().float()
        need_x, need_t = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gxm = gt = efd = None
        with torch.cuda.device(xm.device):
            if need_x:
                efd = torch.empty(N * O, n, L, device=xm.device, dtype=torch.float32)
                _native.call("dl_dwn_prepare_full", tables, efd, N * O, n, ctx.alpha, ctx.beta)
                gxm = torch.empty_like(xm)
            if need_t:
                gt = torch.empty_like(tables)
            if need_x or need_t:
                _native.call("dl_dwn_mapped_bwd", xm, g, efd, gxm, gt, B, N, n, O)
        return gxm, gt, None, None


_IDENTITY_PLANS = {}
FEATURE_MAJOR_MIN_NODES = 64  # below this the row-major kernels are cheaper than two transposes


def _identity_plan(N: int, n: int, out_dim: int, device):
    """Connection plan in which node j reads columns j*n .. j*n+n-1 of a (B, N*n) tensor."""
    from ..layers.fused_ops import ConnectionPlan

    key = (N, n, out_dim, str(device))
    if key not in _IDENTITY_PLANS:
        if len(_IDENTITY_PLANS) > 16:
            _IDENTITY_PLANS.clear()
        mapping = torch.arange(N * n).view(N, n)
        _IDENTITY_PLANS[key] = ConnectionPlan(mapping, N * n, out_dim, torch.device(device))
    return _IDENTITY_PLANS[key]


def dwn_mapped_forward(xm, tables, alpha, beta):
    """Training forward of N nodes on mapped inputs xm (B, N, n) -> (B, N, O) with autograd.

    Wide layers with n <= 6 treat the mapped tensor as N*n input features under the identity map and
    run the feature-major layer kernels (coalesced, shuffle-based EFD look-ups, no atomics); small
    cases and n > 6 use the row-major kernels."""
    B, N, n = xm.shape
    if n <= 6 and N >= FEATURE_MAJOR_MIN_NODES:
        from ..layers.fused_ops import DWNLayerFunction

        plan = _identity_plan(N, n, tables.shape[1], xm.device)
        out = DWNLayerFunction.apply(xm.reshape(B, N * n), tables, plan, alpha, beta)
        return out.reshape(B, N, tables.shape[1])
    return DWNMappedFunction.apply(xm, tables, alpha, beta)


def dwn_mapped_eval(xm, tables):
    """Eval: index from {0,1} inputs, output `table >= 0.5` as fp32 (dwn_node.py:457-483)."""
    _check_cuda(xm, tables)
    xm = xm.contiguous().float()
    tables = tables.detach().contiguous().float()
    B, N, n = xm.shape
    O = tables.shape[1]
    out = torch.empty(B, N, O, device=xm.device, dtype=torch.float32)
    with torch.cuda.device(xm.device):
        _native.call("dl_dwn_mapped_fwd", xm, tables, out, B, N, n, O, 1)
    return out


@register_node("dwn")
class DWNNode(BaseNode):
    """Differentiable weightless node; `luts` has shape (output_dim, 2^input_dim)."""

    def __init__(
        self,
        input_dim: Optional[int] = None,
        output_dim: Optional[int] = None,
        use_cuda: bool = True,
        regularizers: Optional[dict] = None,
        alpha: Optional[float] = None,
        beta: Optional[float] = None,
        clamp_luts: bool = True,
        init_fn: Optional[Callable] = None,
        init_kwargs: Optional[dict] = None,
    ):
        init_kwargs = {} if init_kwargs is None else dict(init_kwargs)
        if "input_dim" not in init_kwargs and input_dim is not None:
            init_kwargs["input_dim"] = input_dim  # residual-style initializers need it
        super().__init__(input_dim=input_dim, output_dim=output_dim, regularizers=regularizers,
                         init_fn=init_fn, init_kwargs=init_kwargs)
        if self.num_inputs > MAX_DWN_INPUT_DIM:
            raise ValueError(f"DWNNode supports input_dim <= {MAX_DWN_INPUT_DIM}, got {self.num_inputs}")
        self.use_cuda = bool(use_cuda)  # accepted for compatibility; there is one (CUDA) path
        self.clamp_luts = clamp_luts
        if alpha is None:
            alpha = default_alpha(self.num_inputs)
            warn_default_value("alpha", alpha, stacklevel=2)
        if beta is None:
            beta = default_beta()
            warn_default_value("beta", beta, stacklevel=2)
        self.register_buffer("alpha", torch.tensor(alpha, dtype=torch.float32))
        self.register_buffer("beta", torch.tensor(beta, dtype=torch.float32))
        self._alpha_f, self._beta_f = float(alpha), float(beta)
        self.luts = nn.Parameter(torch.rand(self.num_outputs, 2 ** self.num_inputs))
        self._apply_init_fn(self.luts, name="luts")

    @classmethod
    def _view_of(cls, layer, index: int) -> "DWNNode":
        """Node object whose `luts` is row `index` of a layer's stacked tables (no own storage)."""
        node = cls.__new__(cls)
        nn.Module.__init__(node)
        node.input_dim, node.output_dim = layer.n, layer.output_dim_per_node
        node.regularizers = layer._node_regularizers
        node.init_fn, node.init_kwargs = layer._node_init_fn, layer._node_init_kwargs
        node.use_cuda, node.clamp_luts = True, True
        node._alpha_f, node._beta_f = layer.alpha, layer.beta
        node.register_buffer("alpha", torch.tensor(layer.alpha, dtype=torch.float32, device=layer.luts.device))
        node.register_buffer("beta", torch.tensor(layer.beta, dtype=torch.float32, device=layer.luts.device))
        node.luts = layer.luts[index]  # a view: in-place edits and gradients reach the layer
        node.training = layer.training
        return node

    def _clamp_luts_if_needed(self) -> None:
        pass  # the reference leaves clamping to the caller (dwn_node.py:426-430)

    def _validate(self, x: torch.Tensor) -> None:
        if x.dim() != 2 or x.shape[1] != self.num_inputs:
            raise ValueError(f"DWNNode expects (batch, {self.num_inputs}) input, got {tuple(x.shape)}")

    def forward_train(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        out = dwn_mapped_forward(x.unsqueeze(1), self.luts.unsqueeze(0), self._alpha_f, self._beta_f)
        return out.squeeze(1)

    def forward_eval(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        return dwn_mapped_eval(x.unsqueeze(1), self.luts.unsqueeze(0)).squeeze(1)

    def forward_with_mapping(self, x: torch.Tensor, mapping_indices: torch.Tensor) -> torch.Tensor:
        """(B, input_size), (layer_size, n) -> (B, layer_size, output_dim): this node's table applied
        at every mapped position (what difflut/nodes/dwn_node.py:485-540 computes)."""
        if mapping_indices.shape[1] != self.num_inputs:
            raise ValueError(
                f"Mapping indices input_dim ({mapping_indices.shape[1]}) doesn't match node's "
                f"input_dim ({self.num_inputs})"
            )
        xm = x[:, mapping_indices.long()]
        tables = self.luts.unsqueeze(0).expand(mapping_indices.shape[0], -1, -1)
        if self.training:
            return dwn_mapped_forward(xm, tables, self._alpha_f, self._beta_f)
        return dwn_mapped_eval(xm, tables)

    def _builtin_regularization(self) -> torch.Tensor:
        return torch.tensor(0.0, device=self.luts.device, requires_grad=False)
