"""Distribution version and API level.

``API_VERSION`` is the level of the public Python surface (it follows the reference's 5.x contract,
``python/rpu_backend/_version.py``) and moves independently of releases.  ``DISTRIBUTION_VERSION`` is read from the
``[project]`` table of ``pyproject.toml`` when running from a source tree, from the installed metadata otherwise."""
from __future__ import annotations

import importlib.metadata as _metadata
import pathlib as _pathlib
import re as _re

API_VERSION = "5.0.0"
_FALLBACK = "0+unknown"


def _from_source_tree():
    pyproject = _pathlib.Path(__file__).resolve().parents[1] / "pyproject.toml"
    try:
        text = pyproject.read_text(encoding="utf-8")
    except OSError:
        return None
    table = _re.search(r"(?ms)^\[project\]\s*$(.*?)(?=^\[|\Z)", text)
    found = _re.search(r"(?m)^version\s*=\s*[\'\"]([^\'\"]+)[\'\"]", table.group(1)) if table else None
    return found.group(1) if found else None


def _resolve() -> str:
    version = _from_source_tree()
    if version:
        return version
    try:
        return _metadata.version("rhinoforge-b200")
    except _metadata.PackageNotFoundError:
        return _FALLBACK


DISTRIBUTION_VERSION = _resolve()

__all__ = ["API_VERSION", "DISTRIBUTION_VERSION"]
