"""Soft input selection of LearnableLayer: `x @ softmax(W / tau, dim=-1).T`.

Reference: difflut/layers/learnable_layer.py:253-255 (F.softmax + torch.matmul).
"""

import torch
import torch.nn.functional as F


def soft_select(x: torch.Tensor, W: torch.Tensor, tau: float) -> torch.Tensor:
    """(B, I), (M, I) -> (B, M) with autograd."""
    if not x.is_cuda:
        raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
    return torch.matmul(x, F.softmax(W / tau, dim=-1).t())
