"""rhinoforge_b200 -- a Blackwell-native inference framework with RhinoForge's public surface.

Importing the package is silent and works without a GPU or the native library: it raises the
open-file limit (best effort), creates the ``torch.rpu`` namespace, binds the four public names
and records the built-in adapter targets without importing any model module.  The same package is
importable as ``rpu_backend``.  Bootstrap order of the reference:
``python/rpu_backend/_bootstrap.py:19-104,183-190``.
"""
from ._bootstrap_env import ensure_nofile_limit as _ensure_nofile_limit

_ensure_nofile_limit()
del _ensure_nofile_limit

import atexit as _atexit  # noqa: E402
import warnings as _warnings  # noqa: E402

import torch as _torch  # noqa: E402

# "rpu" stays a name this package resolves itself (runtime/device.py): registering it as PyTorch's
# PrivateUse1 backend would make torch treat it as the process accelerator and break CUDA
# pinned-memory allocation.
from ._bootstrap_env import configure_hf_cache as _configure_hf_cache  # noqa: E402

_configure_hf_cache()
del _configure_hf_cache

from . import _native  # noqa: E402
from . import _torch_rpu as _trpu  # noqa: E402

_mod = _trpu.install(_torch)
_cpp_loaded = bool(_torch.cuda.is_available() and _native.available())
_cpp_ext = None
if _cpp_loaded:
    try:
        _cpp_ext = _native.lib()
    except Exception:  # noqa: BLE001
        _cpp_loaded, _cpp_ext = False, None

from ._version import DISTRIBUTION_VERSION as __version__  # noqa: E402
from .api.cache import RPUCache  # noqa: E402
from .api.causal_lm import RPUModelForCausalLM  # noqa: E402
from . import graph as _graph  # noqa: E402

_graph.configure_backend(_cpp_ext if _cpp_loaded else None, "<live>" if _cpp_loaded else None)
_graph.install_torch_namespace(_mod)
reset_graph_cache = _graph.reset_graph_cache
_control = _trpu.configure_torch_rpu(_torch, _mod)

from .adapters._manifest import BUILTIN_ADAPTERS as _BUILTINS  # noqa: E402
from .runtime.registry import discover_all as _discover_all  # noqa: E402

_discover_all(_BUILTINS)
del _BUILTINS, _discover_all

# torch.ops.rpu.*: the stand-alone operator surface (kernels are loaded lazily on first call)
from .ops import torch_ops as _torch_ops  # noqa: E402

with _warnings.catch_warnings():
    _warnings.simplefilter("ignore")
    _torch_ops.register()

__all__ = ["__version__", "RPUCache", "RPUModelForCausalLM", "reset_graph_cache"]


def __dir__():
    return list(__all__)


_REMOVED = {
    "build_cache": "use RPUCache.from_model(model, ...)",
    "build_rpu_cache": "use RPUCache.from_model(model, ...)",
    "RPUKVCache": "use RPUCache",
    "convert_linear_weights_inplace": "use rpu_backend.runtime.weights.swizzle_model_inplace",
    "model_converter": "use rpu_backend.runtime.weights.swizzle_model_inplace",
    "Pi05Policy": "use rpu_backend.api.Pi05Policy (lazy import; not at top level)",
    "set_chunk_size": "chunk size is per handle: pass rpu_execution={'prefill': {'chunk_size': n}}",
    "set_spm_mode": "not applicable: activations live in a static device arena",
}
_LAZY_DEBUG = frozenset({"set_debug_level", "get_debug_level", "TRACE"})
_DEPRECATED_GRAPH = {"GraphCache", "GraphSignature", "get_default_graph_cache"}


def __getattr__(name: str):
    if name in _LAZY_DEBUG:
        from .runtime import log as _log
        return getattr(_log, name)
    if name in _DEPRECATED_GRAPH:
        _warnings.warn(f"rpu_backend.{name} is deprecated; use rpu_backend.graph.{name}", DeprecationWarning,
                       stacklevel=2)
        return getattr(_graph, name)
    hint = _REMOVED.get(name)
    if hint:
        raise AttributeError(f"module 'rpu_backend' has no attribute {name!r}; Did you mean: {hint}?")
    raise AttributeError(f"module 'rpu_backend' has no attribute {name!r}")


if _cpp_loaded:
    def _shutdown_at_exit() -> None:
        try:
            _graph.GraphCache.clear_all()
        except Exception:  # noqa: BLE001
            pass
    _atexit.register(_shutdown_at_exit)
