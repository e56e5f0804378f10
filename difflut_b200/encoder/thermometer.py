"""Thermometer encoder backed by the compare-and-pack kernels.

API and arithmetic follow difflut/encoder/thermometer.py:14-128: thresholds are
`min + i*(max-min)/(T+1)` computed with the same torch operations (so the bits are
bit-exact), a bit is 1 iff `x > threshold` (strict), and the flattened column of
(feature f, threshold i) is f*T+i.
"""

import warnings

import torch

from .. import _native
from ..registry import register_encoder
from .base_encoder import BaseEncoder

DEFAULT_THERMOMETER_NUM_BITS: int = 1


@register_encoder("thermometer")
class ThermometerEncoder(BaseEncoder):
    def __init__(self, num_bits: int = DEFAULT_THERMOMETER_NUM_BITS, flatten: bool = True) -> None:
        super().__init__(num_bits=num_bits, flatten=flatten)
        self.thresholds = None  # plain attribute, as in the reference (absent from state_dict)

    def _compute_thresholds(self, x: torch.Tensor) -> torch.Tensor:
        lo = x.min(dim=0)[0]
        hi = x.max(dim=0)[0]
        ticks = torch.arange(1, self.num_bits + 1, device=x.device)
        width = (hi - lo) / (self.num_bits + 1)
        return lo.unsqueeze(-1) + ticks.unsqueeze(0) * width.unsqueeze(-1)

    def fit(self, x) -> "ThermometerEncoder":
        x = self._to_tensor(x)
        if self.num_bits > 32:
            warnings.warn(
                f"ThermometerEncoder: Using {self.num_bits} bits will create many features "
                f"({self.num_bits} per input feature). Consider using fewer bits.",
                UserWarning,
                stacklevel=2,
            )
        self.thresholds = self._compute_thresholds(x)
        self._is_fitted = True
        return self

    # -- kernels ----------------------------------------------------------------------------
    def _prepared(self, x: torch.Tensor):
        """(x as fp32 2-D CUDA rows, thresholds on the same device, leading shape)."""
        if not x.is_cuda:
            raise RuntimeError("difflut_b200.ThermometerEncoder encodes CUDA tensors only (no CPU fallback)")
        lead = x.shape
        x2 = x.reshape(1, -1) if x.dim() == 1 else x.reshape(x.shape[0], -1)
        x2 = x2.contiguous().float()
        thr = self.thresholds.reshape(-1, self.num_bits)
        if thr.device != x.device or thr.dtype != torch.float32:
            thr = thr.to(device=x.device, dtype=torch.float32)
        thr = thr.contiguous()
        if thr.shape[0] != x2.shape[1]:
            raise ValueError(f"encoder was fitted on {thr.shape[0]} features, input has {x2.shape[1]}")
        return x2, thr, lead

    def encode(self, x) -> torch.Tensor:
        """fp32 {0,1} tensor: (B, F*T) if `flatten` else (B, F, T)."""
        self._check_fitted()
        x = self._to_tensor(x)
        x2, thr, lead = self._prepared(x)
        B, F = x2.shape
        out = torch.empty(B, F * self.num_bits, device=x.device, dtype=torch.float32)
        with torch.cuda.device(x.device):
            _native.call("dl_thermo_rows", x2, thr, out, B, F, self.num_bits)
        if self.flatten:
            return out.reshape(-1) if x.dim() == 1 else out
        return out.reshape(*lead, self.num_bits)

    def encode_packed_t(self, x: torch.Tensor) -> torch.Tensor:
        """Bit-packed feature-major encoding: int32 (F*T, Bp/32), bit b%32 of word b//32 = sample b."""
        self._check_fitted()
        x2, thr, _ = self._prepared(x)
        B, F = x2.shape
        Bp = _native.padded_batch(B)
        out = torch.empty(F * self.num_bits, Bp // 32, device=x.device, dtype=torch.int32)
        with torch.cuda.device(x.device):
            _native.call("dl_thermo_pack_t", x2, thr, out, B, F, self.num_bits, Bp)
        return out

    def encode_packed_s(self, x: torch.Tensor) -> torch.Tensor:
        """Bit-packed feature-major encoding in the chunk-interleaved layout the stack kernels read: int32
        (F*T, 32 * ceil(Bp/1024)); bit c + 8r of word w of a 1024-sample block = sample 128c + 4w + r."""
        self._check_fitted()
        x2, thr, _ = self._prepared(x)
        B, F = x2.shape
        Bp = _native.padded_batch(B)
        out = torch.empty(F * self.num_bits, int(_native.lib().dl_swizzled_words(Bp)), device=x.device,
                          dtype=torch.int32)
        with torch.cuda.device(x.device):
            _native.call("dl_thermo_pack_s", x2, thr, out, B, F, self.num_bits, Bp)
        return out

    def encode_packed(self, x: torch.Tensor) -> torch.Tensor:
        """Bit-packed row-major encoding: int32 (B, ceil(F*T/32)), bit c%32 of word c//32 = column c."""
        self._check_fitted()
        x2, thr, _ = self._prepared(x)
        B, F = x2.shape
        out = torch.empty(B, (F * self.num_bits + 31) // 32, device=x.device, dtype=torch.int32)
        with torch.cuda.device(x.device):
            _native.call("dl_thermo_pack_rows", x2, thr, out, B, F, self.num_bits)
        return out

    def binarize(self, x) -> torch.Tensor:
        return self.encode(x)

    def get_thresholds(self, x: torch.Tensor) -> torch.Tensor:
        return self._compute_thresholds(x)

    def __repr__(self) -> str:
        return f"ThermometerEncoder(num_bits={self.num_bits}, flatten={self.flatten})"


@register_encoder("gaussian_thermometer")
class GaussianThermometerEncoder(ThermometerEncoder):
    """Thresholds at Gaussian quantiles of each feature: mean + icdf(i/(T+1)) * std.

    Only `fit` differs from ThermometerEncoder (difflut/encoder/thermometer.py:131-166); encoding
    runs the same compare-and-pack kernels.
    """

    def _compute_thresholds(self, x: torch.Tensor) -> torch.Tensor:
        q = torch.arange(1, self.num_bits + 1, device=x.device).float() / (self.num_bits + 1)
        skews = torch.distributions.Normal(0, 1).icdf(q)
        mean, std = x.mean(dim=0), x.std(dim=0)
        return torch.stack([k * std + mean for k in skews], dim=-1)

    def __repr__(self) -> str:
        return f"GaussianThermometerEncoder(num_bits={self.num_bits}, flatten={self.flatten})"


@register_encoder("distributive_thermometer")
class DistributiveThermometerEncoder(ThermometerEncoder):
    """Thresholds at empirical quantiles of each feature: sorted column value at index
    int(S * i / (T+1)) (difflut/encoder/thermometer.py:169-205)."""

    def _compute_thresholds(self, x: torch.Tensor) -> torch.Tensor:
        ordered = torch.sort(x, dim=0)[0]
        S = ordered.shape[0]
        idx = torch.tensor([int(S * i / (self.num_bits + 1)) for i in range(1, self.num_bits + 1)], device=x.device)
        picked = ordered[idx]  # (T, features...)
        return picked.permute(*range(1, picked.ndim), 0)

    def __repr__(self) -> str:
        return f"DistributiveThermometerEncoder(num_bits={self.num_bits}, flatten={self.flatten})"
