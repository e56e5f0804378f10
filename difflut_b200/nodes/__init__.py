"""Node types of the hot path (registered on import)."""

from .base_node import BaseNode
from .dwn_node import DWNNode
from .dwn_stable_node import DWNStableNode
from .hybrid_node import HybridNode
from .node_config import NodeConfig
from .probabilistic_node import ProbabilisticNode

__all__ = ["BaseNode", "DWNNode", "DWNStableNode", "HybridNode", "ProbabilisticNode", "NodeConfig"]
