"""Error classes raised by the runtime layer itself.

The runtime layer never imports ``api`` or ``adapters`` (dependency direction is
adapters/API -> runtime), so the classes it raises live here and the public
``api.errors`` module re-exports them.  Mirrors the split the reference keeps in
``python/rpu_backend/runtime/__init__.py:18-45``.
"""


class RPUBackendError(Exception):
    """Base class of every error raised by the framework's own surfaces."""


class RPUConfigError(RPUBackendError):
    """Invalid per-instance ``_rpu_*`` attribute or ``rpu_execution`` setting."""


class UnsupportedModelError(RPUBackendError):
    """Architecture is not registered, or its profile is outside the admitted set."""
