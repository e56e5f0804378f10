"""Validated training options of a layer (mirrors difflut/layers/layer_config.py:14-137)."""

from dataclasses import dataclass

GRAD_MODES = ("none", "layerwise", "batchwise")


def check_flip_probability(p) -> None:
    if not isinstance(p, (int, float)) or not (0.0 <= p <= 1.0):
        raise ValueError(
            f"flip_probability must be a float in [0, 1], got {p}. "
            f"Example: flip_probability=0.1 for 10% bit flipping during training."
        )


def check_grad_mode(mode) -> None:
    if mode not in GRAD_MODES:
        raise ValueError(
            f"grad_stabilization must be one of {list(GRAD_MODES)}, got '{mode}'. "
            f"'layerwise': normalize per layer, 'batchwise': normalize per batch sample, 'none': disabled"
        )


def check_positive(name: str, value, hint: str) -> None:
    if not isinstance(value, (int, float)) or value <= 0:
        raise ValueError(f"{name} must be a positive number, got {value}. {hint}")


@dataclass
class LayerConfig:
    flip_probability: float = 0.0
    grad_stabilization: str = "none"
    grad_target_std: float = 1.0
    grad_subtract_mean: bool = False
    grad_epsilon: float = 1e-8

    def __post_init__(self) -> None:
        check_flip_probability(self.flip_probability)
        check_grad_mode(self.grad_stabilization)
        check_positive("grad_target_std", self.grad_target_std, "Example: grad_target_std=1.0 for unit variance")
        check_positive("grad_epsilon", self.grad_epsilon, "Used for numerical stability in variance calculation")

    def copy(self) -> "LayerConfig":
        return LayerConfig(self.flip_probability, self.grad_stabilization, self.grad_target_std,
                           self.grad_subtract_mean, self.grad_epsilon)

    def __repr__(self) -> str:
        parts = []
        if self.flip_probability > 0:
            parts.append(f"flip_probability={self.flip_probability}")
        if self.grad_stabilization != "none":
            parts.append(f"grad_stabilization='{self.grad_stabilization}'")
            parts.append(f"grad_target_std={self.grad_target_std}")
            if self.grad_subtract_mean:
                parts.append(f"grad_subtract_mean={self.grad_subtract_mean}")
        return f"LayerConfig({', '.join(parts)})" if parts else "LayerConfig(default)"


class GroupedInputConfig:
    """Index maps in which every node reads from one input group only.

    Mirrors difflut/layers/layer_config.py:141-221: the `input_size` features form `n_groups`
    consecutive groups (for a convolution: one group per input channel, each of receptive-field size);
    every node draws `bits_per_node` positions inside a group, then the group's offset is added.  The
    same torch CPU generator calls in the same order give the reference's maps bit for bit; the global
    RNG state is saved and restored.
    """

    def __init__(self, n_groups: int, input_size: int, output_trees: int, luts_per_tree: int,
                 bits_per_node: int, seed: int, ensure_full_coverage: bool = True) -> None:
        import torch

        if n_groups < 1:
            raise ValueError(f"n_groups must be >= 1, got {n_groups}. Example: n_groups=4 for 4 input groups.")
        self.n_groups = n_groups
        self.luts_per_tree = luts_per_tree
        total_nodes = output_trees * luts_per_tree
        group_size = input_size // n_groups
        saved = torch.get_rng_state()
        torch.manual_seed(seed)
        within = torch.multinomial(torch.ones((total_nodes, group_size)), num_samples=bits_per_node,
                                   replacement=bits_per_node > group_size)
        if ensure_full_coverage:
            # whole permutations of the groups, then a no-replacement draw for what is left
            cycles, rest = divmod(total_nodes, n_groups)
            picks = [torch.randperm(n_groups) for _ in range(cycles)]
            if rest > 0:
                picks.append(torch.multinomial(torch.ones((n_groups,)), num_samples=rest, replacement=False))
            group_of_node = torch.cat(picks).unsqueeze(1)
        else:
            group_of_node = torch.randint(low=0, high=n_groups, size=(total_nodes, 1))
        self.mapping_indices = within + group_of_node * group_size
        torch.set_rng_state(saved)

    def get_mapping_indices(self, chunk_start: int, chunk_end: int):
        """Rows of the map that belong to trees [chunk_start, chunk_end)."""
        return self.mapping_indices[chunk_start * self.luts_per_tree:chunk_end * self.luts_per_tree, :]
