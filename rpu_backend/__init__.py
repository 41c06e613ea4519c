"""Import-compatible alias: ``rpu_backend`` and every ``rpu_backend.<sub>`` module resolve to the
same module objects as ``rhinoforge_b200`` / ``rhinoforge_b200.<sub>``."""
import importlib
import importlib.abc
import importlib.util
import sys

import rhinoforge_b200 as _impl

_PREFIX, _TARGET = __name__ + ".", "rhinoforge_b200."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self._target = target

    def create_module(self, spec):
        return importlib.import_module(self._target)

    def exec_module(self, module):  # already executed under its real name
        return None


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if found is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real), is_package=found.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

_self = sys.modules[__name__]
for _k in ("__version__", "RPUCache", "RPUModelForCausalLM", "reset_graph_cache", "_cpp_ext", "_cpp_loaded"):
    setattr(_self, _k, getattr(_impl, _k))
__all__ = list(_impl.__all__)


def __getattr__(name):
    return getattr(_impl, name)


def __dir__():
    return list(__all__)
