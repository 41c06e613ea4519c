"""Weight layout API: which way a Linear is partitioned over tensor-parallel ranks, and the packed
(tile-major) device layout of a shard.

The rule is the reference's (``python/rpu_backend/runtime/weights.py:26,97-135,411-544``): q/k/v/gate/up and the
lm_head are COLUMN-partitioned (each rank owns output rows), ``o_proj`` / ``down_proj`` are ROW-partitioned (each
rank owns input columns; the partial products are summed by the all-reduce fused into that GEMM).  "Swizzling"
here means :func:`rhinoforge_b200.ops.kernels.pack_weight`: contiguous 128x64 blocks holding the 128-byte
swizzled shared-memory image, loaded by one bulk copy per block.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Sequence, Tuple

import torch

ROW_PARTITION_NAMES = ("o_proj", "down_proj", "out_proj")
NUM_CORES = 8                      # widest tensor-parallel group (GPUs of one NVSwitch domain)
PARTITION_ROW, PARTITION_COL, PARTITION_HOST = 0, 1, -1


def get_linear_partition(K: int, N: int, dwidth: int = 2, num_cores: int = NUM_CORES, name: str = "") -> int:
    """0 = row partition (split K), 1 = column partition (split N), -1 = leave on the host.

    A Linear stays on the host when neither dimension splits into 16-byte aligned shards."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf in ROW_PARTITION_NAMES:
        return PARTITION_ROW if K % num_cores == 0 and (K // num_cores * dwidth) % 16 == 0 else PARTITION_HOST
    if N % num_cores == 0:
        return PARTITION_COL
    if K % num_cores == 0 and (K // num_cores * dwidth) % 16 == 0:
        return PARTITION_ROW
    return PARTITION_HOST


def shard_linear(weight: torch.Tensor, partition: int, rank: int, world: int) -> torch.Tensor:
    """This rank's shard of a ``[N, K]`` weight under ``partition``."""
    N, K = weight.shape
    if world == 1 or partition == PARTITION_HOST:
        return weight
    if partition == PARTITION_COL:
        per = N // world
        return weight[rank * per:(rank + 1) * per]
    per = K // world
    return weight[:, rank * per:(rank + 1) * per]


def swizzle_linear(weight: torch.Tensor, partition: int = PARTITION_COL, *, rank: int = 0, num_cores: int = 1,
                   sections: int = 1) -> torch.Tensor:
    """Shard (when ``num_cores`` > 1) and pack a Linear weight into the device layout."""
    from ..ops.kernels import pack_weight
    return pack_weight(shard_linear(weight, partition, rank, num_cores).contiguous(), sections)


def partition_plan(named_linears: Iterable[Tuple[str, Tuple[int, int]]], num_cores: int = NUM_CORES) -> Dict[str, int]:
    """``{module name: partition}`` for ``(name, (N, K))`` pairs."""
    return {n: get_linear_partition(K, N, 2, num_cores, n) for n, (N, K) in named_linears}


def convert_model_for_rpu(model: torch.nn.Module, *, num_cores: int = 1, rank: int = 0, skip_names: Iterable[str] = ()) -> dict:
    """Artifact ``{state_dict, partition_info, rpu_converted: True}``: every Linear weight sharded and packed, the
    other tensors untouched.  Tied embeddings are untied first (the lm_head gets its own packed copy)."""
    skip = tuple(skip_names)
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    info: Dict[str, dict] = {}
    for name, mod in model.named_modules():
        if not isinstance(mod, torch.nn.Linear) or any(s in name for s in skip):
            continue
        N, K = mod.weight.shape
        part = get_linear_partition(K, N, mod.weight.element_size(), num_cores, name)
        if part == PARTITION_HOST:
            info[name] = {"partition": part, "shape": (N, K)}
            continue
        w = mod.weight.detach()
        if w.device.type != "cuda":
            w = w.cuda()
        sd[name + ".weight"] = swizzle_linear(w, part, rank=rank, num_cores=num_cores)
        info[name] = {"partition": part, "shape": (N, K), "packed": True}
        mod._rpu_linear_partition = part
    return {"state_dict": sd, "partition_info": info, "rpu_converted": True, "num_cores": num_cores, "rank": rank}


def load_rpu_model(path: str) -> dict:
    """Load an artifact written by ``torch.save(convert_model_for_rpu(...))`` (tensors only)."""
    art = torch.load(path, weights_only=True)
    if not isinstance(art, dict) or not art.get("rpu_converted"):
        raise ValueError(f"{path!r} is not a converted-model artifact")
    return art


_STATUS = {PARTITION_ROW: "row", PARTITION_COL: "col", PARTITION_HOST: "fallback"}


def check_model_rpu_compatible(model: torch.nn.Module, *, tp_degrees: Sequence[int] = (1, 2, 4, 8),
                               decode_rows: int = 64) -> Dict[str, Dict[str, Any]]:
    """What would happen to each ``nn.Linear`` of ``model`` on the accelerator, without touching a weight.

    Per module name: ``in_features``, ``out_features``, ``partition`` / ``status`` at the widest tensor-parallel group
    (``row`` | ``col`` | ``fallback`` - the reference's report, ``python/rpu_backend/runtime/weights.py:654-680``), plus
    ``tp`` - the widest group in ``tp_degrees`` whose shards stay 16-byte aligned - ``shard`` (the ``(N, K)`` one rank
    holds at that width), ``tma_ok`` (K rows start on 16-byte boundaries, the condition for tensor-map loads) and, when
    the native library is built, ``decode_plan``: the GEMM launch plan for ``decode_rows`` tokens on that shard."""
    from ..ops.kernels import gemm_plan
    report: Dict[str, Dict[str, Any]] = {}
    for name, mod in model.named_modules():
        if not isinstance(mod, torch.nn.Linear):
            continue
        K, N = mod.in_features, mod.out_features
        width = mod.weight.element_size() if mod.weight.is_floating_point() else 2
        widest = get_linear_partition(K, N, width, max(tp_degrees), name)
        fit = 1
        for degree in sorted(tp_degrees):
            if get_linear_partition(K, N, width, degree, name) != PARTITION_HOST:
                fit = degree
        part = get_linear_partition(K, N, width, fit, name)
        shard = (N // fit, K) if part == PARTITION_COL else (N, K // fit) if part == PARTITION_ROW else (N, K)
        row = {"in_features": K, "out_features": N, "partition": widest, "status": _STATUS[widest], "tp": fit,
               "shard": shard, "tma_ok": (shard[1] * width) % 16 == 0}
        if row["tma_ok"]:
            plan = gemm_plan(decode_rows, shard[0], shard[1])
            if plan is not None:
                row["decode_plan"] = plan
        report[name] = row
    return report


def print_rpu_compatibility_report(model: torch.nn.Module, **kwargs: Any) -> None:
    """One summary line through the runtime logger (level INFO), then one line per Linear that cannot be accelerated."""
    import logging
    log = logging.getLogger("rpu_backend")
    info = check_model_rpu_compatible(model, **kwargs)
    count = lambda status: sum(1 for r in info.values() if r["status"] == status)
    log.info("Compatibility: %d Linear layers (accelerated: %d, col: %d, row: %d, fallback: %d)", len(info),
             len(info) - count("fallback"), count("col"), count("row"), count("fallback"))
    for name, r in info.items():
        if r["status"] == "fallback" or not r["tma_ok"]:
            log.info("  %s [%d x %d]: %s", name, r["out_features"], r["in_features"],
                     "no aligned tensor-parallel split" if r["tma_ok"] else "K rows are not 16-byte aligned")


__all__ = ["ROW_PARTITION_NAMES", "NUM_CORES", "get_linear_partition", "shard_linear", "swizzle_linear", "partition_plan",
           "convert_model_for_rpu", "load_rpu_model", "check_model_rpu_compatible", "print_rpu_compatibility_report"]
