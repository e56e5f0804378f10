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
