"""GroupSum: contiguous groups of node outputs summed into class scores.

Same constructor, validation and warnings as the reference module
(difflut/utils/modules.py:20-163); CUDA inputs run the `dl_groupsum_rows` kernels.
"""

import warnings
from typing import Optional

import torch
import torch.nn as nn

from .. import _native
from .warnings import warn_default_value

DEFAULT_GROUPSUM_K: int = 1
DEFAULT_GROUPSUM_TAU: float = 1.0
DEFAULT_GROUPSUM_USE_RANDPERM: bool = False


class _GroupSumFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, tau):
        x = x.contiguous().float()
        B, F = x.shape
        out = torch.empty(B, k, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            _native.call("dl_groupsum_rows", x, out, B, F, k, tau)
        ctx.dims = (B, F, k, tau)
        return out

    @staticmethod
    def backward(ctx, gout):
        B, F, k, tau = ctx.dims
        gout = gout.contiguous().float()
        gx = torch.empty(B, F, device=gout.device, dtype=torch.float32)
        with torch.cuda.device(gout.device):
            _native.call("dl_groupsum_rows_bwd", gout, gx, B, F, k, tau)
        return gx, None, None


class GroupSum(nn.Module):
    """(B, F) -> (B, k): class c sums columns [c*g, (c+1)*g), g = ceil(F/k), divided by tau."""

    def __init__(self, k: Optional[int] = None, tau: Optional[float] = None,
                 use_randperm: Optional[bool] = None) -> None:
        super().__init__()
        if k is None:
            k = DEFAULT_GROUPSUM_K
            warn_default_value("k (GroupSum)", k, stacklevel=2)
        if tau is None:
            tau = DEFAULT_GROUPSUM_TAU
            warn_default_value("tau (GroupSum)", tau, stacklevel=2)
        if use_randperm is None:
            use_randperm = DEFAULT_GROUPSUM_USE_RANDPERM
            warn_default_value("use_randperm (GroupSum)", use_randperm, stacklevel=2)
        self.k, self.tau, self.use_randperm = k, tau, use_randperm
        if not isinstance(self.k, int) or self.k <= 0:
            raise ValueError(f"k must be a positive integer, got {self.k}")
        if not isinstance(self.tau, (int, float)) or self.tau <= 0:
            raise ValueError(f"tau must be a positive number, got {self.tau}")

    def _validate_input_dim(self, x: torch.Tensor) -> None:
        if x.dim() != 2:
            raise ValueError(
                f"GroupSum expects 2D input (batch_size, num_features), but got shape {x.shape} "
                f"with {x.dim()} dimensions."
            )
        batch_size, num_features = x.shape
        if batch_size == 0:
            raise ValueError(f"GroupSum requires non-empty batch, got batch_size={batch_size}")
        if num_features == 0:
            raise ValueError(f"GroupSum requires non-zero features, got num_features={num_features}.")
        if num_features < self.k:
            warnings.warn(
                f"GroupSum input has fewer features ({num_features}) than output groups ({self.k}). "
                f"Some groups will receive zero features.",
                UserWarning,
                stacklevel=3,
            )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._validate_input_dim(x)
        if self.use_randperm:
            x = x[:, torch.randperm(x.shape[-1], device=x.device)]
        num_features = x.shape[-1]
        if num_features % self.k != 0:
            pad = self.k - (num_features % self.k)
            warnings.warn(
                f"GroupSum: Input has {num_features} features which is not divisible by k={self.k}. "
                f"Adding {pad} zero-padded features.",
                UserWarning,
                stacklevel=2,
            )
        if not x.is_cuda:
            raise RuntimeError("difflut_b200.GroupSum runs on CUDA tensors only (no CPU fallback)")
        # zero padding changes no sum: the kernel clips the last group at F instead
        return _GroupSumFn.apply(x, self.k, float(self.tau))
