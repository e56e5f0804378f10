"""Probabilistic node: expectation of a sigmoid-weighted table under independent Bernoulli inputs.

Public surface and arithmetic follow difflut/nodes/probabilistic_node.py:153-335:
training output = sum_a sigma(raw[a]/max(T,1e-6)) * prod_j (a_j ? x_j : 1-x_j) (LSB-first
patterns), eval output = hard lookup of the sigmoid table thresholded at >= 0.5.  Parity
target is the reference's PyTorch (autograd) path: inputs are not clamped and the input
gradient is the product rule.  The kernels live in `csrc/prob.cu`.
"""

from typing import Any, Callable, Dict, Optional, Tuple

import torch
import torch.nn as nn

from .. import _native
from ..registry import register_node
from .base_node import BaseNode

DEFAULT_PROBABILISTIC_TEMPERATURE: float = 1.0
DEFAULT_PROBABILISTIC_EVAL_MODE: str = "expectation"
DEFAULT_PROBABILISTIC_USE_CUDA: bool = True
MAX_PROB_INPUT_DIM: int = 6


def _identity_map(N: int, n: int, device) -> torch.Tensor:
    return torch.arange(N * n, device=device, dtype=torch.int32).reshape(N, n).contiguous()


class ProbMappedFunction(torch.autograd.Function):
    """N nodes on already-mapped inputs: xm (B,N,n), raw (N,2^n,O) -> (B,N,O).

    Counterpart of ProbabilisticFunction (difflut/nodes/probabilistic_node.py:39-129) for N nodes.
    The mapped tensor is viewed as N*n independent input features with the identity map, so the
    feature-major layer kernels are reused unchanged.
    """

    @staticmethod
    def forward(ctx, xm, raw, temperature):
        if not (xm.is_cuda and raw.is_cuda):
            raise RuntimeError("difflut_b200 probabilistic kernels run on CUDA tensors only (no CPU fallback)")
        xm = xm.contiguous().float()
        raw = raw.contiguous().float()
        B, N, n = xm.shape
        O = raw.shape[2]
        if n > MAX_PROB_INPUT_DIM:
            raise RuntimeError(f"ProbabilisticNode kernels support input_dim <= {MAX_PROB_INPUT_DIM}, got {n}")
        Bp = _native.padded_batch(B)
        with torch.cuda.device(xm.device):
            x_t = torch.empty(N * n, Bp, device=xm.device, dtype=torch.float32)
            _native.call("dl_f32_rows_to_t", xm.reshape(B, N * n), x_t, B, N * n, Bp)
            idmap = _identity_map(N, n, xm.device)
            out_t = torch.empty(N * O, Bp, device=xm.device, dtype=torch.float32)
            _native.call("dl_prob_fwd_t", x_t, idmap, raw, temperature, out_t, N, n, O, Bp)
            out = torch.empty(B, N * O, device=xm.device, dtype=torch.float32)
            _native.call("dl_f32_t_to_rows", out_t, out, B, N * O, Bp)
        ctx.save_for_backward(x_t, raw, idmap)
        ctx.temperature, ctx.dims = float(temperature), (B, N, n, O, Bp)
        return out.reshape(B, N, O)

    @staticmethod
    def backward(ctx, g):
        x_t, raw, idmap = ctx.saved_tensors
        B, N, n, O, Bp = ctx.dims
        need_x, need_r = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        gxm = None
        with torch.cuda.device(g.device):
            g_t = torch.empty(N * O, Bp, device=g.device, dtype=torch.float32)
            _native.call("dl_f32_rows_to_t", g.contiguous().float().reshape(B, N * O), g_t, B, N * O, Bp)
            graw = torch.empty_like(raw)
            gxm_t = torch.empty(N * n, Bp, device=g.device, dtype=torch.float32) if need_x else None
            _native.call("dl_prob_bwd_t", x_t, idmap, raw, ctx.temperature, g_t, 1, 1.0, graw, gxm_t, N, n, O, B, Bp)
            if need_x:
                gxm = torch.empty(B, N * n, device=g.device, dtype=torch.float32)
                _native.call("dl_f32_t_to_rows", gxm_t, gxm, B, N * n, Bp)
                gxm = gxm.reshape(B, N, n)
        return gxm, (graw if need_r else None), None


def prob_mapped_forward(xm, raw, temperature):
    return ProbMappedFunction.apply(xm, raw, temperature)


def prob_mapped_eval(xm, raw, temperature):
    """Eval: index from {0,1} inputs into sigma(raw/T); output `>= 0.5` as fp32
    (probabilistic_node.py:302-328).  sigma(z) >= 0.5 iff z >= 0, so the lookup runs on raw/T."""
    from .dwn_node import dwn_mapped_eval

    t = max(float(temperature), 1e-6)
    # DWN eval kernel thresholds at 0.5: feed it sigma(raw/T) laid out (N, O, 2^n)
    tables = torch.sigmoid(raw.detach().float() / t).permute(0, 2, 1).contiguous()
    return dwn_mapped_eval(xm, tables)


@register_node("probabilistic")
class ProbabilisticNode(BaseNode):
    """`raw_weights` has shape (2^input_dim, output_dim)."""

    def __init__(
        self,
        input_dim: Optional[int] = None,
        output_dim: Optional[int] = None,
        init_fn: Optional[Callable[[torch.Tensor], None]] = None,
        init_kwargs: Optional[Dict[str, Any]] = None,
        regularizers: Optional[Dict[str, Tuple[Callable, float, Dict[str, Any]]]] = None,
        temperature: float = DEFAULT_PROBABILISTIC_TEMPERATURE,
        eval_mode: str = DEFAULT_PROBABILISTIC_EVAL_MODE,
        use_cuda: bool = DEFAULT_PROBABILISTIC_USE_CUDA,
    ) -> None:
        super().__init__(input_dim=input_dim, output_dim=output_dim, regularizers=regularizers,
                         init_fn=init_fn, init_kwargs=init_kwargs)
        self.register_buffer("temperature", torch.tensor(float(temperature)))
        self._temperature_f = float(temperature)
        assert eval_mode in {"expectation", "deterministic", "threshold"}, "Invalid eval_mode"
        self.eval_mode = eval_mode
        self.use_cuda = bool(use_cuda)  # accepted for compatibility; there is one (CUDA) path
        self.raw_weights = nn.Parameter(torch.randn(2 ** self.input_dim, self.output_dim))
        self._apply_init_fn(self.raw_weights, name="raw_weights")
        self.register_buffer("binary_combinations", self.binary_patterns(self.input_dim, "cpu"))

    @staticmethod
    def binary_patterns(n: int, device) -> torch.Tensor:
        """(2^n, n) fp32, row a = bits of a, LSB first (probabilistic_node.py:227-234)."""
        a = torch.arange(2 ** n, device=device)
        return ((a[:, None] >> torch.arange(n, device=device)[None, :]) & 1).float()

    @classmethod
    def _view_of(cls, layer, index: int) -> "ProbabilisticNode":
        """Node object whose `raw_weights` is row `index` of a layer's stacked tables."""
        node = cls.__new__(cls)
        nn.Module.__init__(node)
        node.input_dim, node.output_dim = layer.n, layer.output_dim_per_node
        node.regularizers = layer._node_regularizers
        node.init_fn, node.init_kwargs = layer._node_init_fn, layer._node_init_kwargs
        node.eval_mode, node.use_cuda = layer.eval_mode, True
        dev = layer.raw_weights.device
        node._temperature_f = layer.temperature
        node.register_buffer("temperature", torch.tensor(layer.temperature, device=dev))
        node.register_buffer("binary_combinations", cls.binary_patterns(layer.n, dev))
        node.raw_weights = layer.raw_weights[index]
        node.training = layer.training
        return node

    @property
    def weights(self) -> torch.Tensor:
        return torch.sigmoid(self.raw_weights / self.temperature.clamp(min=1e-6))

    def _binary_to_index(self, x_binary: torch.Tensor) -> torch.Tensor:
        powers = 2 ** torch.arange(self.input_dim, device=x_binary.device, dtype=torch.float32)
        return (x_binary * powers).sum(dim=-1).long() if x_binary.dim() > 1 else (x_binary * powers).sum().long()

    def _validate(self, x: torch.Tensor) -> None:
        if x.dim() != 2 or x.shape[1] != self.input_dim:
            raise ValueError(f"ProbabilisticNode expects (batch, {self.input_dim}) input, got {tuple(x.shape)}")

    def forward_train(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        out = prob_mapped_forward(x.unsqueeze(1), self.raw_weights.unsqueeze(0), self._temperature_f)
        return out.squeeze(1)

    def forward_eval(self, x: torch.Tensor) -> torch.Tensor:
        self._validate(x)
        return prob_mapped_eval(x.unsqueeze(1), self.raw_weights.unsqueeze(0), self._temperature_f).squeeze(1)

    def _builtin_regularization(self) -> torch.Tensor:
        return torch.tensor(0.0, device=self.raw_weights.device)

    def extra_repr(self) -> str:
        return f"input_dim={self.input_dim}, output_dim={self.output_dim}"
