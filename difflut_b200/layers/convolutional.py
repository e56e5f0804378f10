"""Convolutional LUT layer: one small tree of LUT layers per output channel, applied to every patch.

Constructor, sub-layer structure and output follow difflut/layers/convolutional.py:13-266: patches of
`in_channels * kh * kw` features (nn.Unfold order) go through `out_channels` trees whose layers have
`n^depth, n^(depth-1), ..., 1` nodes; the first tree layers are built in chunks of `chunk_size` trees
(`first_layer_chunks`), the rest per tree (`trees[t][l]`), every one an instance of `layer_type` built
with that type's default seed, so maps, parameters and state-dict keys are the reference's.

Execution differs.  When `layer_type` is RandomLayer with one of the package's stacked node types, all
trees of a depth level run as ONE layer: their index maps are merged into one block-diagonal map (tree t
reads columns t*h .. t*h+h-1 of the level below) and their parameters are concatenated, so a forward is
`depth + 1` layer kernels instead of `out_channels * depth + chunks` small ones.  For node types that only
read `x >= 0.5` (DWN, DWNStable; every stacked type in eval mode) the patches are never materialised:
bits are packed straight from the image (`dl_unfold_pack_t`), the tree levels exchange one bit per
activation (`DWNStackFunction`: bit-sliced forward, one fused backward kernel per level) and the input
gradient is folded straight back (`dl_fold_t`).  Any other layer / node class keeps the reference's loop over sub-layers on patches
produced by `dl_unfold_rows`.
"""

from typing import Optional, Type

import torch
import torch.nn as nn

from ..nodes.node_config import NodeConfig
from ..registry import register_convolutional_layer
from .base_layer import LUTLayerMixin
from .fused_ops import (ConnectionPlan, DWNStackFunction, PatchFunction, PatchGeometry, StackOptions,
                        dwn_levels_eval)
from .layer_config import GroupedInputConfig, LayerConfig
from .random_layer import RandomLayer


class ConvolutionConfig:
    """Geometry and tree shape of a ConvolutionalLayer (difflut/layers/convolutional.py:13-41)."""

    def __init__(self, tree_depth: int = 2, in_channels=None, out_channels=None, receptive_field=5,
                 stride=1, padding=0, chunk_size: int = 32, seed: int = 42):
        assert in_channels is not None, "in_channels must be specified"
        assert out_channels is not None, "out_channels must be specified"
        self.tree_depth = tree_depth
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.receptive_field = receptive_field
        self.stride = stride
        self.padding = padding
        self.chunk_size = chunk_size
        self.seed = seed


@register_convolutional_layer("convolutional")
class ConvolutionalLayer(LUTLayerMixin, nn.Module):
    """(B, in_channels, H, W) -> (B, out_channels, OH, OW)."""

    def __init__(
        self,
        convolution_config: ConvolutionConfig,
        node_type: Type[nn.Module],
        node_kwargs: NodeConfig,
        layer_type: Type[nn.Module],
        n_inputs_per_node: int = 6,
        layer_config: Optional[LayerConfig] = None,
        flip_probability: Optional[float] = None,
        grad_stabilization: Optional[str] = None,
        grad_target_std: Optional[float] = None,
        grad_subtract_mean: Optional[bool] = None,
        grad_epsilon: Optional[float] = None,
        grouped_connections: bool = False,
        ensure_full_coverage: bool = False,
    ):
        super().__init__()
        self._init_lut_layer_mixin(layer_config, flip_probability, grad_stabilization, grad_target_std,
                                   grad_subtract_mean, grad_epsilon)
        cfg = convolution_config
        self.tree_depth = cfg.tree_depth
        self.in_channels = cfg.in_channels
        self.out_channels = cfg.out_channels
        self.receptive_field = self._pair(cfg.receptive_field)
        self.input_size = self.in_channels * self.receptive_field[0] * self.receptive_field[1]
        self.stride = self._pair(cfg.stride)
        self.padding = self._pair(cfg.padding)
        self.node_type = node_type
        self.layer_type = layer_type
        self.n_inputs_per_node = n_inputs_per_node
        self.seed = cfg.seed
        self.chunk_size = min(cfg.chunk_size, self.out_channels)
        self.hidden_layers = [n_inputs_per_node ** (self.tree_depth - i) for i in range(self.tree_depth + 1)]
        h0 = self.hidden_layers[0]

        grouped = None
        if grouped_connections:
            assert self.input_size % self.in_channels == 0, "Input size must be divisible by number of groups."
            grouped = GroupedInputConfig(n_groups=self.in_channels, input_size=self.input_size,
                                         output_trees=self.out_channels, luts_per_tree=h0,
                                         bits_per_node=n_inputs_per_node, seed=self.seed,
                                         ensure_full_coverage=ensure_full_coverage)

        self.first_layer_chunks = nn.ModuleList()
        for start in range(0, self.out_channels, self.chunk_size):
            stop = min(start + self.chunk_size, self.out_channels)
            self.first_layer_chunks.append(layer_type(
                input_size=self.input_size, output_size=h0 * (stop - start), node_type=node_type,
                node_kwargs=node_kwargs,
                mapping_indices=grouped.get_mapping_indices(start, stop) if grouped else None))

        self.trees = nn.ModuleList()
        for _ in range(self.out_channels):
            tree, width = nn.ModuleList(), h0
            for out_width in self.hidden_layers[1:]:
                tree.append(layer_type(input_size=width, output_size=out_width, node_type=node_type,
                                       node_kwargs=node_kwargs))
                width = out_width
            self.trees.append(tree)
        self._level_plans = None
        self._merge_ok = None

    @staticmethod
    def _pair(x):
        return (x, x) if isinstance(x, int) else tuple(x)

    def __repr__(self) -> str:
        return (
            f"ConvolutionalLUTLayer(\n"
            f"  receptive_field={self.receptive_field}, stride={self.stride}, padding={self.padding}\n"
            f"  in_channels={self.in_channels}, out_channels={self.out_channels}\n"
            f"  tree_architecture={self.hidden_layers}\n"
            f"  node_type={self.node_type}, layer_type={self.layer_type}\n"
            f"  n_inputs_per_node={self.n_inputs_per_node}, tree_depth={self.tree_depth}\n"
            f"  total_trees={len(self.trees)}, chunk_size={self.chunk_size}, "
            f"num_chunks={len(self.first_layer_chunks)}\n"
            f")"
        )

    # ------------------------------------------------------------------ merged levels
    def _level_layers(self):
        """Sub-layers per depth level, in tree order."""
        levels = [list(self.first_layer_chunks)]
        for l in range(self.tree_depth):
            levels.append([tree[l] for tree in self.trees])
        return levels

    def _mergeable(self) -> bool:
        """All sub-layers are RandomLayers of one stacked node type (fixed at construction: checked once)."""
        if self._merge_ok is None:
            subs = [layer for level in self._level_layers() for layer in level]
            self._merge_ok = all(type(s) is RandomLayer and s._stacked is not None and s.output_dim_per_node == 1
                                 and s._stacked == subs[0]._stacked for s in subs)
        return self._merge_ok

    def _apply(self, fn, *args, **kwargs):
        self._level_plans = None  # buffers are replaced by .to() / .cuda(): rebuild the merged maps
        return super()._apply(fn, *args, **kwargs)

    def _load_from_state_dict(self, *args, **kwargs):
        self._level_plans = None  # the sub-layers' maps may be overwritten
        return super()._load_from_state_dict(*args, **kwargs)

    def _plans(self, device):
        """One ConnectionPlan per depth level: the sub-layers' maps side by side, each tree's map shifted
        to that tree's block of the level below.  Built once per device; moving the module or loading a
        state dict drops it (a map edited in place afterwards needs `conv._level_plans = None`)."""
        if self._level_plans is not None and self._level_plans[0] == str(device):
            return self._level_plans[1]
        plans = []
        for depth, level in enumerate(self._level_layers()):
            if depth == 0:
                rows = [s._mapping_indices.long() for s in level]
                width = self.input_size
            else:
                below = self.hidden_layers[depth - 1]
                rows = [s._mapping_indices.long() + t * below for t, s in enumerate(level)]
                width = below * self.out_channels
            plans.append(ConnectionPlan(torch.cat(rows, dim=0), width, 1, device))
        self._level_plans = (str(device), plans)
        return plans

    @staticmethod
    def _level_params(level):
        """Concatenated parameters of a level's sub-layers (autograd routes gradients back to each)."""
        if len(level) == 1:
            return level[0]._own_params()
        return tuple(torch.cat(parts, dim=0) for parts in zip(*(s._own_params() for s in level)))

    def _forward_merged(self, x: torch.Tensor, geom: PatchGeometry, flip: bool) -> torch.Tensor:
        levels = self._level_layers()
        plans = self._plans(x.device)
        proto = levels[0][0]
        hard_eval = not self.training and proto._stacked in ("dwn", "dwn_stable", "hybrid") and proto.n <= 6
        if hard_eval:
            tables = []
            for level in levels:
                p = self._level_params(level)[0]
                tables.append(p if proto._stacked == "dwn" else torch.sigmoid(p))
            return dwn_levels_eval(x, list(zip(tables, plans)), geom)
        bits_only = self.training and proto._stacked in ("dwn", "dwn_stable") and proto.n <= 6
        source = geom
        if flip and bits_only:
            # the nodes only read `patch >= 0.5`: flip the packed patch bits instead of materialising patches
            if self.flip_probability < 0.05:
                # the reference's sparse rule: an exact number of the B*P x (C*kh*kw) patch entries flips
                numel = geom.S * geom.F
                flip_spec = (float(self.flip_probability), 0, self._draw_flip_positions(numel, x.device))
            else:
                flip_spec = (float(self.flip_probability), self._draw_seed())
            source = StackOptions(geom, flip=flip_spec)
            h = x
        elif flip:
            h = self._apply_bit_flip(PatchFunction.apply(x, geom))
            geom = source = None
        else:
            h = x
        if bits_only:
            # all levels as one bit-packed pipeline: no fp32 activations between the tree levels
            stable = proto._stacked == "dwn_stable"
            params = [self._level_params(level) for level in levels]
            tables = [torch.sigmoid(p[0]) if stable else p[0] for p in params]
            spec = [(plan, 0.0 if stable else proto.alpha, 0.0 if stable else proto.beta,
                     p[1].detach().float() if stable else None) for plan, p in zip(plans, params)]
            return DWNStackFunction.apply(h, spec, source, *tables)
        for level, plan in zip(levels, plans):
            h = level[0]._apply_plan(h, plan, self._level_params(level), geom)
            geom = None
        return h

    def _forward_loop(self, patches: torch.Tensor) -> torch.Tensor:
        """The reference's schedule (convolutional.py:214-240) for arbitrary layer / node classes."""
        S = patches.shape[0]
        out = torch.empty(S, self.out_channels, device=patches.device)
        t = 0
        h0 = self.hidden_layers[0]
        for chunk in self.first_layer_chunks:
            first = chunk(patches)
            trees_here = first.shape[1] // h0
            first = first.view(S, trees_here, h0)
            for local in range(trees_here):
                h = first[:, local, :]
                for layer in self.trees[t]:
                    h = layer(h)
                out[:, t] = h.squeeze(-1)
                t += 1
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 4 or x.shape[1] != self.in_channels:
            raise ValueError(
                f"ConvolutionalLayer expects (batch, {self.in_channels}, H, W) input, got {tuple(x.shape)}"
            )
        if not x.is_cuda:
            raise RuntimeError("difflut_b200 layers run on CUDA tensors only (no CPU fallback)")
        geom = PatchGeometry(x.shape, self.receptive_field, self.stride, self.padding)
        flip = self.training and self.flip_probability > 0.0
        if self._mergeable():
            rows = self._forward_merged(x, geom, flip)
        else:
            patches = PatchFunction.apply(x, geom)
            if flip:
                patches = self._apply_bit_flip(patches)
            rows = self._forward_loop(patches)
        out = rows.view(geom.B, geom.P, self.out_channels).transpose(1, 2)
        out = out.view(geom.B, self.out_channels, geom.OH, geom.OW)
        if self.grad_stabilization != "none" and self.training and out.requires_grad:
            def rescale(grad):
                return self._apply_gradient_stabilization(grad.reshape(grad.shape[0], -1)).view(grad.shape)

            out.register_hook(rescale)
        return out
