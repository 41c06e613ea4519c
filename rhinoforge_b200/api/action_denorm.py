"""Config-driven action de-normalisation: a policy emits actions in a normalised space; deployment maps each
contiguous group of action dimensions back to physical units and, for delta actions, adds the matching state.
Nothing about a robot is hard-coded: groups, their normalisation kind and the statistics all come from
configuration (reference: ``python/rpu_backend/api/action_denorm.py:50-300``).

Kinds: ``meanstd`` ``x*(std+eps)+mean``; ``std`` ``x*(std+eps)``; ``minmax`` / ``bounds_98`` / ``bounds_99``
``(clip(x,-1,1)+1)/2*(hi-lo+eps)+lo`` with (min,max) / (q02,q98) / (q01,q99); the ``*_woclip`` forms skip the
clip; ``identity``.  ``eps = 1e-6`` as in the normaliser that produced the statistics.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Mapping, Optional, Sequence

import numpy as np
import torch

EPS = 1e-6
_RANGE_KEYS = {"minmax": ("min", "max"), "minmax_woclip": ("min", "max"), "bounds_98": ("q02", "q98"),
               "bounds_98_woclip": ("q02", "q98"), "bounds_99": ("q01", "q99"), "bounds_99_woclip": ("q01", "q99")}
_REQUIRED = {"meanstd": ("mean", "std"), "std": ("std",), "identity": (), **_RANGE_KEYS}
SUPPORTED_NORM_TYPES = frozenset(_REQUIRED)


@dataclass(frozen=True)
class ActionGroup:
    key: str
    dim: int
    norm_type: str
    subtract_state: bool = False       # delta action: physical = unnormalised + state
    state_key: Optional[str] = None


@dataclass
class ActionDenormalizer:
    groups: Sequence[ActionGroup]
    norm_stats: Mapping[str, Mapping[str, np.ndarray]]
    _offsets: list = field(default_factory=list)

    def __post_init__(self):
        if not self.groups:
            raise ValueError("action de-normalizer requires at least one action group")
        acc = 0
        for g in self.groups:
            if isinstance(g.dim, bool) or not isinstance(g.dim, (int, np.integer)) or int(g.dim) <= 0:
                raise ValueError(f"action group {g.key!r} has invalid dim {g.dim!r}; dim must be a positive integer")
            if g.norm_type not in SUPPORTED_NORM_TYPES:
                raise ValueError(f"action group {g.key!r} has norm_type {g.norm_type!r}; supported: {sorted(SUPPORTED_NORM_TYPES)}")
            if g.norm_type != "identity":
                if g.key not in self.norm_stats:
                    raise KeyError(f"norm_stats is missing key {g.key!r}")
                for name in _REQUIRED[g.norm_type]:
                    if name not in self.norm_stats[g.key]:
                        raise KeyError(f"norm_stats[{g.key!r}] is missing {name!r} for norm_type {g.norm_type!r}")
                    v = np.asarray(self.norm_stats[g.key][name], dtype=np.float64)
                    if v.ndim not in (1, 2) or v.shape[-1] != int(g.dim):
                        raise ValueError(f"{g.key}.{name} has shape {v.shape}, expected [..., {int(g.dim)}]")
            if g.subtract_state and not g.state_key:
                raise ValueError(f"delta action group {g.key!r} needs a state_key")
            self._offsets.append((acc, acc + int(g.dim)))
            acc += int(g.dim)
        self.total_dim = acc

    @classmethod
    def from_files(cls, groups: Sequence[Mapping], stats_json: str) -> "ActionDenormalizer":
        with open(stats_json, "r", encoding="utf-8") as f:
            raw = json.load(f)
        stats = raw.get("norm_stats", raw)
        return cls([ActionGroup(**g) for g in groups], {k: {n: np.asarray(v) for n, v in s.items()} for k, s in stats.items()})

    def _unnorm(self, g: ActionGroup, x: np.ndarray) -> np.ndarray:
        if g.norm_type == "identity":
            return x
        s = {k: np.asarray(v, dtype=np.float64) for k, v in self.norm_stats[g.key].items()}
        if g.norm_type == "meanstd":
            return x * (s["std"] + EPS) + s["mean"]
        if g.norm_type == "std":
            return x * (s["std"] + EPS)
        lo, hi = (s[k] for k in _RANGE_KEYS[g.norm_type])
        if not g.norm_type.endswith("_woclip"):
            x = np.clip(x, -1.0, 1.0)
        return (x + 1.0) / 2.0 * (hi - lo + EPS) + lo

    def __call__(self, actions, state: Optional[Mapping[str, np.ndarray]] = None) -> np.ndarray:
        """``actions [H, >= total_dim]`` (tensor or array) -> physical ``[H, total_dim]`` float64."""
        a = actions.detach().float().cpu().numpy() if torch.is_tensor(actions) else np.asarray(actions)
        a = a.astype(np.float64)
        if a.ndim != 2 or a.shape[1] < self.total_dim:
            raise ValueError(f"actions must be [horizon, >= {self.total_dim}], got {a.shape}")
        out = np.empty((a.shape[0], self.total_dim), dtype=np.float64)
        for g, (b, e) in zip(self.groups, self._offsets):
            v = self._unnorm(g, a[:, b:e])
            if g.subtract_state:
                if state is None or g.state_key not in state:
                    raise KeyError(f"delta action group {g.key!r} needs state[{g.state_key!r}]")
                v = v + np.asarray(state[g.state_key], dtype=np.float64).reshape(1, -1)[:, :e - b]
            out[:, b:e] = v
        return out


__all__ = ["ActionGroup", "ActionDenormalizer", "SUPPORTED_NORM_TYPES", "EPS"]
