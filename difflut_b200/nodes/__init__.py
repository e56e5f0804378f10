"""Node types of the hot path (registered on import)."""

from .base_node import BaseNode
from .dwn_node import DWNNode
from .node_config import NodeConfig
from .probabilistic_node import ProbabilisticNode

__all__ = ["BaseNode", "DWNNode", "ProbabilisticNode", "NodeConfig"]
