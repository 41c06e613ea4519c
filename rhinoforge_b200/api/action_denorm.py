"""Config-driven action de-normalisation: a policy emits actions in a normalised space; deployment maps each
contiguous group of action dimensions back to physical units and, for delta actions, adds the matching state.
Nothing about a robot is hard-coded: groups, their normalisation kind and the statistics all come from
configuration (reference: ``python/rpu_backend/api/action_denorm.py:50-300``).

Kinds: ``meanstd`` ``x*(std+eps)+mean``; ``std`` ``x*(std+eps)``; ``minmax`` / ``bounds_98`` / ``bounds_99``
``(x+1)/2*(hi-lo+eps)+lo`` with (min,max) / (q02,q98) / (q01,q99); ``identity``.  The clip of the ``minmax`` /
``bounds_*`` kinds belongs to the forward (normalising) direction only: the inverse never clips, so a kind and its
``*_woclip`` twin de-normalise identically, exactly as in the reference (``_unnormalize_group``).  Statistics are
``[dim]`` or per-step ``[chunk, dim]``; the latter are cut to the action horizon.  ``eps = 1e-6`` as in the
normaliser that produced the statistics.
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
                    if v.ndim == 2 and v.shape[0] == 0:
                        raise ValueError(f"{g.key}.{name} has an empty horizon")
                    if not np.isfinite(v).all():
                        raise ValueError(f"{g.key}.{name} contains non-finite statistics")
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

    # ---- constructors from configuration files (reference: ``api/action_denorm.py:204-320``) -------------------
    @classmethod
    def from_spec(cls, norm_stats_path: str, groups: Sequence[ActionGroup]) -> "ActionDenormalizer":
        """The caller names the ordered groups; statistics come from ``norm_stats_path`` (a JSON object, optionally
        nested under ``"norm_stats"``)."""
        return cls(list(groups), _read_stats(norm_stats_path))

    @classmethod
    def from_norm_json(cls, norm_stats_path: str, *, default_norm_type: str = "meanstd",
                       robot_config=None) -> "ActionDenormalizer":
        """Diagnostic constructor: one group per ``action.*`` key of the statistics file, in file order, width taken
        from the last axis of its ``mean``, all of one normalisation kind.  The file cannot prove joint order or kind,
        so robot-facing code should use :meth:`from_training_config` or an explicit spec."""
        stats = _read_stats(norm_stats_path)
        delta = _delta_flags(robot_config)
        groups = []
        for key, st in stats.items():
            if not key.startswith("action."):
                continue
            mean = np.asarray(st["mean"])
            if mean.ndim == 0:
                raise ValueError(f"{key}.mean must have an action dimension")
            groups.append(ActionGroup(key, int(mean.shape[-1]), default_norm_type, bool(delta.get(key, False)),
                                      "observation.state." + key[len("action."):]))
        if not groups:
            raise ValueError(f"no 'action.*' keys found in {norm_stats_path}")
        return cls(groups, stats)

    @classmethod
    def from_training_config(cls, norm_stats_path: str, training_config, *, robot_config=None) -> "ActionDenormalizer":
        """Groups from the training configuration (a mapping or a YAML path): ``data.joints`` gives the order and width
        of each joint group (entries ``{name: dim}`` or their ``repr``), ``data.norm_type`` the kind of each
        (``{name: kind}``).  A group without an explicit kind is refused rather than treated as identity.  The optional
        robot configuration only contributes the ``subtract_state`` (delta action) flags."""
        cfg = _mapping_or_yaml(training_config)
        data = cfg["data"] if "data" in cfg else cfg
        widths = [(name, int(dim)) for entry in data["joints"] for name, dim in _pairs(entry)]
        kinds = {name: kind for entry in data["norm_type"] for name, kind in _pairs(entry)}
        unnamed = [name for name, _ in widths if name not in kinds]
        if unnamed:
            raise ValueError(f"training config is missing explicit norm_type entries for action groups {unnamed}; "
                             "refusing to guess identity")
        delta = _delta_flags(robot_config)
        groups = [ActionGroup(f"action.{name}", dim, kinds[name], bool(delta.get(f"action.{name}", False)),
                              f"observation.state.{name}") for name, dim in widths]
        return cls(groups, _read_stats(norm_stats_path))

    @property
    def real_dim(self) -> int:
        """Action columns that are real degrees of freedom; a model pads its action vector beyond them."""
        return self.total_dim

    def unapply(self, action_norm, state=None) -> torch.Tensor:
        """``[H, D]`` or ``[1, H, D]`` normalised actions (``D >= real_dim``) -> physical ``[H, real_dim]`` fp32.

        ``state`` is the flat physical proprioception vector laid out like the action groups; it is required exactly
        when some group is a delta action, and each such group adds its own slice of it.  Non-finite inputs or results
        are refused - they must never reach an actuator."""
        a = action_norm.detach().float().cpu() if torch.is_tensor(action_norm) else torch.as_tensor(action_norm, dtype=torch.float32)
        if a.dim() == 3:
            if a.shape[0] != 1:
                raise ValueError(f"expected batch 1, got {tuple(a.shape)}")
            a = a[0]
        if a.dim() != 2:
            raise ValueError(f"action must be [H, D], got {tuple(a.shape)}")
        if a.shape[1] < self.real_dim:
            raise ValueError(f"action has {a.shape[1]} dims < real_dim {self.real_dim}")
        if not bool(torch.isfinite(a).all()):
            raise ValueError("normalized action contains non-finite values")
        x = a[:, :self.real_dim].numpy().astype(np.float64)
        flat = None if state is None else torch.as_tensor(state, dtype=torch.float64).reshape(-1).numpy()
        out = np.empty_like(x)
        for g, (b, e) in zip(self.groups, self._offsets):
            v = self._unnorm(g, x[:, b:e])
            if g.subtract_state:
                if flat is None:
                    raise ValueError(f"group {g.key!r} is a delta action (subtract_state=True) but no state was "
                                     "provided to unapply().")
                if flat.size < e:
                    raise ValueError(f"state has {flat.size} dims, but group {g.key!r} ends at {e}")
                if not np.isfinite(flat[b:e]).all():
                    raise ValueError(f"state slice for group {g.key!r} is non-finite")
                v = v + flat[b:e]
            out[:, b:e] = v
        result = torch.from_numpy(out).to(torch.float32)
        if not bool(torch.isfinite(result).all()):
            raise ValueError("de-normalized action contains non-finite values")
        return result

    def _stat(self, key: str, name: str, horizon: int) -> np.ndarray:
        """Statistic ``name`` of group ``key`` for an action of ``horizon`` steps: per-step ``[chunk, dim]`` tables
        are cut to the first ``horizon`` rows (a shorter table is an error), ``[dim]`` vectors broadcast."""
        s = np.asarray(self.norm_stats[key][name], dtype=np.float64)
        if s.ndim == 2:
            if s.shape[0] < horizon:
                raise ValueError(f"{key}.{name} horizon {s.shape[0]} < action horizon {horizon}")
            s = s[:horizon]
        return s

    def _unnorm(self, g: ActionGroup, x: np.ndarray) -> np.ndarray:
        if g.norm_type == "identity":
            return x
        H = x.shape[0]
        if g.norm_type == "meanstd":
            return x * (self._stat(g.key, "std", H) + EPS) + self._stat(g.key, "mean", H)
        if g.norm_type == "std":
            return x * (self._stat(g.key, "std", H) + EPS)
        lo, hi = (self._stat(g.key, k, H) for k in _RANGE_KEYS[g.norm_type])
        return (x + 1.0) / 2.0 * (hi - lo + EPS) + lo      # no clip on the way back (see the module docstring)

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


def _read_stats(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    return raw.get("norm_stats", raw)


def _mapping_or_yaml(x):
    if isinstance(x, Mapping):
        return x
    import yaml
    with open(x, "r", encoding="utf-8") as f:
        return yaml.safe_load(f)


def _pairs(entry):
    """``{name: value}`` entries of a training config come as mappings or as their ``repr`` strings."""
    import ast
    return (ast.literal_eval(entry) if isinstance(entry, str) else dict(entry)).items()


def _delta_flags(robot_config) -> dict:
    """``{action key: subtract_state}`` from a robot configuration's ``actions: [{key: {subtract_state: bool}}]``."""
    if robot_config is None:
        return {}
    flags = {}
    for entry in _mapping_or_yaml(robot_config).get("actions", None) or []:
        if isinstance(entry, Mapping):
            for key, info in entry.items():
                if isinstance(info, Mapping) and "subtract_state" in info:
                    flags[key] = bool(info["subtract_state"])
    return flags


__all__ = ["ActionGroup", "ActionDenormalizer", "SUPPORTED_NORM_TYPES", "EPS"]
