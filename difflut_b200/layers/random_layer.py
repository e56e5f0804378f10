"""RandomLayer: fixed seeded connectivity feeding N LUT nodes.

Constructor, index-map generation and accessors follow difflut/layers/random_layer.py:123-356
(the map is drawn with the same torch CPU generator calls, so it is bit-identical for a given
seed).  With DWN / Probabilistic nodes the forward is a single fused kernel; `get_mapping`
still returns the materialised (B, N, n) tensor for callers that want it.
"""

from typing import Optional, Type

import torch
import torch.nn as nn

from ..nodes.node_config import NodeConfig
from ..registry import register_layer
from .base_layer import BaseLUTLayer
from .fused_ops import GatherFunction, ProbLayerFunction
from .layer_config import LayerConfig

DEFAULT_RANDOM_LAYER_SEED: int = 42
FAST_PATH_MAX_N: int = 6


def draw_random_mapping(input_size: int, output_size: int, n: int, seed: int,
                        ensure_full_input_coverage: bool) -> torch.Tensor:
    """(N, n) int16/int32 index map; the global CPU RNG state is saved and restored.

    Coverage mode concatenates `randperm(input_size)` cycles plus a no-replacement remainder;
    otherwise every node draws n inputs with `multinomial` (random_layer.py:207-256).
    """
    state = torch.get_rng_state()
    torch.manual_seed(seed)
    dtype = torch.int16 if input_size < 32768 else torch.int32
    if not ensure_full_input_coverage:
        idx = torch.multinomial(torch.ones((output_size, input_size)), num_samples=n,
                                replacement=n > input_size).to(dtype)
    else:
        total = output_size * n
        cycles, rest = divmod(total, input_size)
        chunks = [torch.randperm(input_size) for _ in range(cycles)]
        if rest > 0:
            chunks.append(torch.multinomial(torch.ones(input_size), num_samples=rest, replacement=False))
        idx = torch.cat(chunks).reshape(output_size, n).to(dtype)
    torch.set_rng_state(state)
    return idx


@register_layer("random")
class RandomLayer(BaseLUTLayer):
    def __init__(
        self,
        input_size: int,
        output_size: int,
        node_type: Type[nn.Module],
        node_kwargs: NodeConfig,
        seed: Optional[int] = DEFAULT_RANDOM_LAYER_SEED,
        layer_config: Optional[LayerConfig] = None,
        flip_probability: Optional[float] = None,
        grad_stabilization: Optional[str] = None,
        grad_target_std: Optional[float] = None,
        grad_subtract_mean: Optional[bool] = None,
        grad_epsilon: Optional[float] = None,
        ensure_full_input_coverage: bool = True,
        mapping_indices: Optional[torch.Tensor] = None,
    ) -> None:
        self.seed = seed
        super().__init__(input_size=input_size, output_size=output_size, node_type=node_type,
                         node_kwargs=node_kwargs, layer_config=layer_config,
                         flip_probability=flip_probability, grad_stabilization=grad_stabilization,
                         grad_target_std=grad_target_std, grad_subtract_mean=grad_subtract_mean,
                         grad_epsilon=grad_epsilon)
        self._init_mapping(ensure_full_input_coverage=ensure_full_input_coverage,
                           mapping_indices=mapping_indices)

    def _init_mapping(self, ensure_full_input_coverage: bool = True,
                      mapping_indices: Optional[torch.Tensor] = None) -> None:
        if mapping_indices is not None:
            dtype = torch.int16 if self.input_size < 32768 else torch.int32
            idx = mapping_indices.to(dtype=dtype)
        else:
            idx = draw_random_mapping(self.input_size, self.output_size, self.n, self.seed,
                                      ensure_full_input_coverage)
        self.register_buffer("_mapping_indices", idx)

    def _plan(self, device):
        return self._plan_for(self._mapping_indices, device, "random")

    def get_mapping(self, x: torch.Tensor) -> torch.Tensor:
        return GatherFunction.apply(x, self._plan(x.device))

    def get_mapping_indices(self):
        return self._mapping_indices

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._validate_input_dims(x)
        return self._apply_plan(x, self._plan(x.device))

    def forward_groupsum(self, x: torch.Tensor, k: int, tau: float = 1.0) -> torch.Tensor:
        """Probabilistic layer fused with the following GroupSum(k, tau): (B, I) -> (B, k) logits,
        equal to GroupSum(k, tau)(layer(x)) without materialising the (B, N) node outputs."""
        self._validate_input_dims(x)
        if not (self._stacked == "probabilistic" and self.n <= FAST_PATH_MAX_N and self.training):
            raise RuntimeError("forward_groupsum needs a training-mode layer of ProbabilisticNode with n <= 6")
        return ProbLayerFunction.apply(x, self.raw_weights, self._plan(x.device), self.temperature, int(k), float(tau))

    def get_mapping_matrix(self) -> torch.Tensor:
        return self._mapping_indices.long()

    def extra_repr(self) -> str:
        flip = f", flip_prob={self.flip_probability}" if self.flip_probability > 0 else ""
        grad = f", grad_stab={self.grad_stabilization}" if self.grad_stabilization != "none" else ""
        return (f"input_size={self.input_size}, output_size={self.output_size}, "
                f"n={self.n}, seed={self.seed}, mapping=random{flip}{grad}")
