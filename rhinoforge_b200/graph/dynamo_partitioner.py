"""Cut a traced FX graph into runs that can be stream-captured and nodes that have to talk to the host.

A CUDA graph records kernel launches; it cannot contain an operation whose *result the host reads* (``.item()``,
``.tolist()``, ``nonzero`` and other data-dependent output shapes) or that moves data between host and device through
pageable memory - such a call synchronises, which is illegal during stream capture, and on replay the host would see
the value of the recording run anyway.  :func:`partition_for_capture` walks the nodes in order, labels each one, and
splits the module wherever the label flips, producing a chain ``[capturable run, host node(s), capturable run, ...]``
whose pieces the Dynamo backend wraps individually.  The reference partitions for the analogous reason - operations
that must observe data materialised by the preceding recorded run (``python/rpu_backend/graph/dynamo_partitioner.py:1-60``).

Labelling is conservative: when in doubt a node is sent to the host side, because an unnecessary cut costs one launch
boundary while a wrongly captured node produces stale values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.fx
from torch.fx.passes.split_module import split_module

# method / function names whose result lives on the host or whose output shape depends on data
HOST_NAMES = frozenset({"item", "tolist", "numpy", "cpu", "nonzero", "masked_select", "unique", "unique_consecutive",
                        "_local_scalar_dense", "argwhere", "bincount", "is_nonzero", "equal", "allclose", "pin_memory",
                        "print"})


def _target_name(node: torch.fx.Node) -> str:
    t = node.target
    if isinstance(t, str):
        return t
    name = getattr(t, "__name__", None) or str(t)
    return name.split(".")[0] if name.startswith("aten") else name.rsplit(".", 1)[-1]


def _moves_off_device(node: torch.fx.Node) -> bool:
    """``.to("cpu")`` / ``.to(device=...)`` / ``_to_copy(device=...)`` with a host target."""
    if _target_name(node) not in ("to", "_to_copy"):
        return False
    wanted = [node.kwargs.get("device")] + [a for a in node.args[1:] if isinstance(a, (str, torch.device))]
    return any(w is not None and torch.device(w).type == "cpu" for w in wanted)


def default_is_capturable(node: torch.fx.Node) -> bool:
    """False for nodes that synchronise with, or deliver data to, the host."""
    if node.op not in ("call_function", "call_method", "call_module"):
        return True
    if node.op == "call_module":
        return True
    return _target_name(node) not in HOST_NAMES and not _moves_off_device(node)


@dataclass(frozen=True)
class Segment:
    name: str                # attribute name of the sub-module in ``Partitioned.module``
    capturable: bool
    n_nodes: int


class Partitioned:
    """The split module plus the order and kind of its segments."""

    def __init__(self, module: torch.fx.GraphModule, segments: List[Segment]):
        self.module = module
        self.segments = segments
        self._index = {s.name: i for i, s in enumerate(segments)}

    def run(self, args: Sequence[Any],
            call: Optional[Callable[[int, Segment, Callable[..., Any], Sequence[Any]], Any]] = None) -> Any:
        """Interpret the top-level graph, handing every segment call to ``call(index, segment, fn, args)`` (default:
        just run it).  Anything else in the top-level graph (``getitem`` on a segment's tuple output) runs as it is."""
        env: Dict[torch.fx.Node, Any] = {}
        feed = iter(args)
        look = lambda a: torch.fx.node.map_arg(a, lambda n: env[n])
        for node in self.module.graph.nodes:
            if node.op == "placeholder":
                env[node] = next(feed)
            elif node.op == "output":
                return look(node.args[0])
            elif node.op == "call_module" and node.target in self._index:
                i = self._index[node.target]
                fn, seg_args = getattr(self.module, node.target), look(node.args)
                env[node] = fn(*seg_args) if call is None else call(i, self.segments[i], fn, seg_args)
            elif node.op == "call_function":
                env[node] = node.target(*look(node.args), **look(node.kwargs))
            elif node.op == "get_attr":
                env[node] = getattr(self.module, node.target)
            else:  # pragma: no cover - split_module emits nothing else at the top level
                raise RuntimeError(f"unexpected top-level node {node.format_node()}")
        raise RuntimeError("graph without an output node")


def partition_for_capture(gm: torch.fx.GraphModule,
                          is_capturable: Optional[Callable[[torch.fx.Node], bool]] = None) -> Partitioned:
    """Split ``gm`` at every flip between capturable and host nodes; the pieces keep the original order."""
    pred = is_capturable or default_is_capturable
    part_of: Dict[torch.fx.Node, int] = {}
    kinds: List[bool] = []
    for node in gm.graph.nodes:
        if node.op in ("placeholder", "output", "get_attr"):
            continue
        ok = bool(pred(node))
        if not kinds or kinds[-1] != ok:
            kinds.append(ok)
        part_of[node] = len(kinds) - 1
    if not kinds:
        return Partitioned(gm, [])
    split = split_module(gm, None, lambda n: part_of[n], keep_original_order=True)
    segments: List[Segment] = []
    for node in split.graph.nodes:
        if node.op == "call_module" and str(node.target).startswith("submod_"):
            idx = int(str(node.target).rsplit("_", 1)[1])
            sub = getattr(split, node.target)
            body = sum(1 for n in sub.graph.nodes if n.op not in ("placeholder", "output", "get_attr"))
            segments.append(Segment(str(node.target), kinds[idx], body))
    return Partitioned(split, segments)


__all__ = ["partition_for_capture", "default_is_capturable", "Partitioned", "Segment", "HOST_NAMES"]
