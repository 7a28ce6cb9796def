"""B200-native kernels for the RefactorGraph transformer-decoder hot path (C ABI in include/rg_b200.h)."""
from . import capi  # noqa: F401
