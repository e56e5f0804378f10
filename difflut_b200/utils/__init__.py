"""Utility modules (GroupSum) and warning helpers."""

from .modules import GroupSum
from .warnings import (
    ConfigurationWarning,
    CUDAWarning,
    DefaultValueWarning,
    DiffLUTWarning,
    PerformanceWarning,
    configure_warnings,
    disable_all_warnings,
    disable_cuda_warnings,
    enable_all_warnings,
    enable_strict_mode,
    suppress_warnings,
    warn_default_value,
)
