"""Public error hierarchy (reference: ``python/rpu_backend/api/errors.py:1-40``).

``RPUBackendError`` is the base; ``SPMExhaustionError`` keeps its name for API
compatibility and is raised here when a plan exceeds the static device arena or
the paged KV pool.
"""
from ..runtime.errors import RPUBackendError, RPUConfigError, UnsupportedModelError


class RPUUnsupportedDtypeError(RPUBackendError):
    """The requested dtype is not supported on the selected path."""


class RPUSingleHandleError(RPUBackendError):
    """A second live model or policy handle was requested in one process."""


class SPMExhaustionError(RPUBackendError):
    """The execution plan does not fit the activation arena / KV pool."""


class WeightShapeMismatchError(RPUBackendError):
    """A weight tensor violates the layout constraints of its adapter."""


__all__ = [
    "RPUBackendError",
    "RPUConfigError",
    "UnsupportedModelError",
    "RPUUnsupportedDtypeError",
    "RPUSingleHandleError",
    "SPMExhaustionError",
    "WeightShapeMismatchError",
]
