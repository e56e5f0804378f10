"""difflut_b200: B200-native kernels behind DiffLUT's registry / node / layer / encoder API.

Import layout mirrors the reference package (`difflut`): `REGISTRY`, the `register_*`
decorators, `BaseNode`, `BaseLUTLayer`, `BaseEncoder`, and the sub-packages `nodes`, `layers`,
`encoder`, `utils`.  Importing the package registers "dwn", "probabilistic", "random",
"learnable" and "thermometer".  All arithmetic runs in the CUDA library built from `csrc/`
(`python -m difflut_b200.build`); there is no CPU path.
"""

from .registry import (
    REGISTRY,
    register_convolutional_layer,
    register_encoder,
    register_initializer,
    register_layer,
    register_node,
    register_regularizer,
)
from .encoder.base_encoder import BaseEncoder
from .nodes.base_node import BaseNode
from .layers.base_layer import BaseLUTLayer
from . import encoder, layers, nodes, utils  # noqa: F401  (registration side effects)

__version__ = "0.1.0"

__all__ = [
    "REGISTRY",
    "register_node",
    "register_layer",
    "register_convolutional_layer",
    "register_encoder",
    "register_initializer",
    "register_regularizer",
    "BaseNode",
    "BaseLUTLayer",
    "BaseEncoder",
]
