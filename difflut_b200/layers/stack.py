"""Consecutive DWN layers behind one module, executed as one bit-packed pipeline.

The reference chains layers with `nn.Sequential`; every layer then takes and returns fp32 rows
(difflut/layers/random_layer.py:306-340), which for a 16 000-node layer at batch 8192 is half a gigabyte
written and read back per layer and direction.  A DWN layer only looks at `input >= 0.5`, so `DWNStack`
runs the same layers (it holds the caller's layer objects: same parameters, maps and state dict) through
`DWNStackFunction`: one bit per activation between layers, table values only at the last one, one fused
backward kernel per layer.  Outputs and gradients are those of the layer-by-layer chain.  It is a normal
autograd module: any loss, any torch optimiser.
"""

from typing import Optional, Sequence

import torch
import torch.nn as nn

from ..encoder.thermometer import ThermometerEncoder
from ..utils.modules import GroupSum
from .fused_ops import DWNStackFunction, PackedInput, StackOptions, dwn_levels_eval
from .random_layer import RandomLayer


class DWNStack(nn.Module):
    """`DWNStack(layers)(x)` equals `nn.Sequential(*layers)(x)` for RandomLayer layers of DWNNode /
    DWNStableNode with n <= 6 and output_dim 1.  With `encoder`, the module takes raw features and packs
    the thermometer bits itself (`DWNStack(layers, encoder)(x)` equals `Sequential(*layers)(encoder(x))`;
    the raw features then receive no gradient, as the encoder has none).  With `groupsum` (a GroupSum
    without random permutation) the class sums are fused into the last layer's kernels and the module
    returns the (B, k) logits of `groupsum(Sequential(*layers)(x))` without writing the last layer's
    (B, N) outputs in training mode."""

    def __init__(self, layers: Sequence[RandomLayer], encoder: Optional[ThermometerEncoder] = None,
                 groupsum: Optional[GroupSum] = None):
        super().__init__()
        layers = list(layers)
        if not layers:
            raise ValueError("DWNStack needs at least one layer")
        width = None
        for l in layers:
            ok = (type(l) is RandomLayer and l._stacked in ("dwn", "dwn_stable") and l.n <= 6
                  and l.output_dim_per_node == 1)
            if not ok:
                raise ValueError("DWNStack takes RandomLayer layers of DWNNode / DWNStableNode with n <= 6 and "
                                 "output_dim 1")
            if l.flip_probability > 0.0 or l.grad_stabilization != "none":
                raise ValueError("DWNStack does not apply flip_probability / grad_stabilization between its "
                                 "bit-packed layers; call such layers one by one")
            if width is not None and l.input_size != width:
                raise ValueError(f"layer input_size {l.input_size} does not match the {width} outputs feeding it")
            width = l.output_size
        self.layers = nn.ModuleList(layers)
        self.encoder = encoder  # plain attribute, as thresholds are in the reference's encoders
        if groupsum is not None and groupsum.use_randperm:
            raise ValueError("DWNStack cannot fuse GroupSum(use_randperm=True)")
        self.groupsum = groupsum

    def _spec(self, device):
        spec, tables = [], []
        for l in self.layers:
            plan = l._plan(device)
            if l._stacked == "dwn":
                spec.append((plan, l.alpha, l.beta, None))
                tables.append(l.luts)
            else:
                spec.append((plan, 0.0, 0.0, l.gradient_scale.detach().float()))
                tables.append(torch.sigmoid(l.raw_luts))
        return spec, tables

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
        spec, tables = self._spec(x.device)
        source = None
        if self.encoder is not None:
            batch = x.shape[0]
            interleaved = self.training and self.groupsum is not None
            x = self.encoder.encode_packed_s(x) if interleaved else self.encoder.encode_packed_t(x)
            source = PackedInput(batch, interleaved)
        else:
            self.layers[0]._validate_input_dims(x)
        if self.training:
            head = (self.groupsum.k, self.groupsum.tau) if self.groupsum is not None else None
            return DWNStackFunction.apply(x, spec, StackOptions(source, head=head), *tables)
        out = dwn_levels_eval(x, [(t, s[0]) for t, s in zip(tables, spec)], source)
        return out if self.groupsum is None else self.groupsum(out)
