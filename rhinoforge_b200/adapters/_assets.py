"""Checks of on-disk assets before they are loaded: an optional ``{path: sha256}`` manifest pins every file an adapter
reads (reference behaviour: ``python/rpu_backend/adapters/navdp/runtime.py:256-266``, the manifest checks of the
standalone builders)."""
from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Iterable, Mapping, Optional, Union

PathLike = Union[str, Path]


def sha256_of(path: PathLike, chunk: int = 1 << 22) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                return h.hexdigest()
            h.update(b)


def verify_asset_manifest(paths: Iterable[PathLike], manifest: Optional[Mapping[PathLike, str]]) -> None:
    """With a manifest, every path must be listed (by resolved path or file name) and hash to the listed digest."""
    if manifest is None:
        return
    table = {}
    for k, v in manifest.items():
        table[str(Path(k).expanduser().resolve()) if Path(k).is_absolute() or Path(k).exists() else str(k)] = v.lower()
    for p in paths:
        rp = Path(p).expanduser().resolve()
        want = table.get(str(rp), table.get(rp.name))
        if want is None:
            raise ValueError(f"{rp} is not listed in the asset manifest")
        got = sha256_of(rp)
        if got != want:
            raise ValueError(f"{rp}: SHA-256 {got} does not match the manifest's {want}")


__all__ = ["sha256_of", "verify_asset_manifest"]
