"""Global component registry with the reference's names and behaviour (difflut/registry.py:11-458).

Six tables (nodes, layers, convolutional layers, encoders, initializers, regularizers), a
decorator per table, `get_*` raising ValueError with the list of known names, `list_*`, and
`build_*` shortcuts.  Initializers / regularizers are stored lower-case; a name ending in
`_init` / `_regularizer` is also reachable without the suffix.
"""

import warnings
from typing import Any, Callable, Dict, List, Optional, Type


class Registry:
    _KINDS = ("node", "layer", "convolutional_layer", "encoder")

    def __init__(self) -> None:
        self._nodes: Dict[str, Type] = {}
        self._layers: Dict[str, Type] = {}
        self._convolutional_layers: Dict[str, Type] = {}
        self._encoders: Dict[str, Type] = {}
        self._initializers: Dict[str, Callable] = {}
        self._regularizers: Dict[str, Callable] = {}

    # -- class tables -------------------------------------------------------------------
    def _register_class(self, table: Dict[str, Type], label: str, lister: str, name: Optional[str]):
        def decorator(cls: Type) -> Type:
            key = name if name is not None else cls.__name__
            if key in table:
                warnings.warn(
                    f"{label} '{key}' is already registered and will be overwritten. "
                    f"Check existing registrations with registry.{lister}().",
                    UserWarning,
                    stacklevel=2,
                )
            table[key] = cls
            return cls

        return decorator

    @staticmethod
    def _lookup(table: Dict[str, Any], label: str, plural: str, name: str):
        if name not in table:
            raise ValueError(f"{label} '{name}' not found. Available {plural}: {list(table.keys())}")
        return table[name]

    def register_node(self, name: Optional[str] = None) -> Callable:
        return self._register_class(self._nodes, "Node", "list_nodes", name)

    def get_node(self, name: str) -> Type:
        return self._lookup(self._nodes, "Node", "nodes", name)

    def list_nodes(self) -> List[str]:
        return list(self._nodes.keys())

    def register_layer(self, name: Optional[str] = None) -> Callable:
        return self._register_class(self._layers, "Layer", "list_layers", name)

    def get_layer(self, name: str) -> Type:
        return self._lookup(self._layers, "Layer", "layers", name)

    def list_layers(self) -> List[str]:
        return list(self._layers.keys())

    def register_convolutional_layer(self, name: Optional[str] = None) -> Callable:
        return self._register_class(
            self._convolutional_layers, "Convolutional layer", "list_convolutional_layers", name
        )

    def get_convolutional_layer(self, name: str) -> Type:
        return self._lookup(self._convolutional_layers, "Convolutional layer", "convolutional layers", name)

    def list_convolutional_layers(self) -> List[str]:
        return list(self._convolutional_layers.keys())

    def register_encoder(self, name: Optional[str] = None) -> Callable:
        return self._register_class(self._encoders, "Encoder", "list_encoders", name)

    def get_encoder(self, name: str) -> Type:
        return self._lookup(self._encoders, "Encoder", "encoders", name)

    def list_encoders(self) -> List[str]:
        return list(self._encoders.keys())

    # -- function tables ----------------------------------------------------------------
    def _register_function(self, table: Dict[str, Callable], label: str, suffix: str, name: Optional[str]):
        def decorator(func: Callable) -> Callable:
            key = (name if name is not None else func.__name__).lower()
            keys = [key]
            if key.endswith(suffix):
                keys.append(key[: -len(suffix)])
            for k in keys:
                if k in table:
                    warnings.warn(
                        f"{label} '{k}' is already registered and will be overwritten.",
                        UserWarning,
                        stacklevel=2,
                    )
                table[k] = func
            return func

        return decorator

    def register_initializer(self, name: Optional[str] = None) -> Callable:
        return self._register_function(self._initializers, "Initializer", "_init", name)

    def get_initializer(self, name: str) -> Callable:
        return self._lookup_ci(self._initializers, "Initializer", "initializers", name)

    def list_initializers(self) -> List[str]:
        return sorted(self._initializers.keys())

    def register_regularizer(self, name: Optional[str] = None) -> Callable:
        return self._register_function(self._regularizers, "Regularizer", "_regularizer", name)

    def get_regularizer(self, name: str) -> Callable:
        return self._lookup_ci(self._regularizers, "Regularizer", "regularizers", name)

    def list_regularizers(self) -> List[str]:
        return sorted(self._regularizers.keys())

    @staticmethod
    def _lookup_ci(table, label, plural, name):
        """Case-insensitive lookup (function tables are stored lower-case)."""
        if name.lower() not in table:
            raise ValueError(f"{label} '{name}' not found. Available {plural}: {list(table.keys())}")
        return table[name.lower()]

    # -- builders -------------------------------------------------------------------------
    def build_node(self, name: str, **kwargs) -> Any:
        return self.get_node(name)(**kwargs)

    def build_layer(self, name: str, **kwargs) -> Any:
        return self.get_layer(name)(**kwargs)

    def build_convolutional_layer(self, name: str, **kwargs) -> Any:
        return self.get_convolutional_layer(name)(**kwargs)

    def build_encoder(self, name: str, **kwargs) -> Any:
        return self.get_encoder(name)(**kwargs)

    def list_all(self) -> Dict[str, List[str]]:
        return {
            "nodes": self.list_nodes(),
            "layers": self.list_layers(),
            "convolutional_layers": self.list_convolutional_layers(),
            "encoders": self.list_encoders(),
            "initializers": self.list_initializers(),
            "regularizers": self.list_regularizers(),
        }

    def __repr__(self) -> str:
        counts = {k: len(v) for k, v in self.list_all().items()}
        body = ",\n".join(f"  {k}={v}" for k, v in counts.items())
        return f"Registry(\n{body}\n)"


REGISTRY = Registry()

register_node = REGISTRY.register_node
register_layer = REGISTRY.register_layer
register_convolutional_layer = REGISTRY.register_convolutional_layer
register_encoder = REGISTRY.register_encoder
register_initializer = REGISTRY.register_initializer
register_regularizer = REGISTRY.register_regularizer
