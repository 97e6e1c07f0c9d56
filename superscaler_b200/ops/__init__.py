"""Kernels and differentiable ops (native sm_100a extension + CPU restatements for tests)."""
from . import native  # noqa: F401
from . import functional  # noqa: F401
