"""Public error hierarchy: everything derives from ``RPUBackendError`` (names as in the reference,
``python/rpu_backend/api/errors.py:1-40``, so that ``except`` clauses written against it keep working).

``SPMExhaustionError`` keeps its historical name; here it means that an execution plan exceeds the static
activation arena or the paged KV pool.
"""
from ..runtime.errors import RPUBackendError, RPUConfigError, UnsupportedModelError

_DERIVED = {
    "RPUUnsupportedDtypeError": "The requested dtype is not supported on the selected path.",
    "RPUSingleHandleError": "A second live model or policy handle was requested in one process.",
    "SPMExhaustionError": "The execution plan does not fit the activation arena / KV pool.",
    "WeightShapeMismatchError": "A weight tensor violates the layout constraints of its adapter.",
}
for _name, _doc in _DERIVED.items():
    globals()[_name] = type(_name, (RPUBackendError,), {"__doc__": _doc, "__module__": __name__})
del _name, _doc

__all__ = ["RPUBackendError", "RPUConfigError", "UnsupportedModelError", *_DERIVED]
