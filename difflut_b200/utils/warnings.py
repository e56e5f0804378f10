"""Warning categories and helpers; names match the reference (difflut/utils/warnings.py:26-147)
because user code filters on them."""

import warnings
from typing import Any, Optional, Type


class DiffLUTWarning(UserWarning):
    """Base category for package-specific warnings."""


class PerformanceWarning(RuntimeWarning):
    """Something works but is slower than it could be."""


class ConfigurationWarning(UserWarning):
    """A configuration is legal but probably not what was intended."""


class DefaultValueWarning(ConfigurationWarning):
    """An optional parameter was left out and its default is used."""


class CUDAWarning(PerformanceWarning):
    """CUDA availability / kernel selection notices."""


def warn_default_value(param_name: str, param_value: Any, stacklevel: int = 2) -> None:
    warnings.warn(
        f"Parameter '{param_name}' was not provided, using default value: {param_value}",
        category=DefaultValueWarning,
        stacklevel=stacklevel + 1,
    )


def configure_warnings(action: str = "default", category: Optional[Type[Warning]] = None,
                       module_pattern: str = "difflut") -> None:
    if category is None:
        warnings.filterwarnings(action, module=module_pattern)
    else:
        warnings.filterwarnings(action, category=category, module=module_pattern)


def suppress_warnings(func: Any) -> Any:
    def wrapper(*args: Any, **kwargs: Any) -> Any:
        with warnings.catch_warnings():
            warnings.filterwarnings("ignore", module="difflut")
            return func(*args, **kwargs)

    return wrapper


def enable_all_warnings() -> None:
    configure_warnings("always")


def disable_all_warnings() -> None:
    configure_warnings("ignore")


def disable_cuda_warnings() -> None:
    configure_warnings("ignore", category=PerformanceWarning)


def enable_strict_mode() -> None:
    configure_warnings("error")
