"""Shared helpers of the causal-decoder runtimes: the bounded prefill planner and the graph-signature keys.

The reference plans every multi-token forward as ``(execution_len, chunk_size)``: how many rows really run (the
logical rows plus optional inert causal tail rows) and in launches of how many rows
(``python/rpu_backend/runtime/decoder.py:276-448``), and folds the chunk policy and the resume position into the graph
signature (``:108-153``).  On this hardware prefill is a packed variable-length launch, so every length is legal and
padding never buys a cheaper plan by itself; the planner is kept because the *contract* is public - adapters declare an
execution-length alignment, callers may pin ``chunk_size`` and ``padding_rows`` through ``rpu_execution``, and
``model._rpu_last_execution_plan`` reports what was resolved.

``plan_bounded_prefill_execution`` is resolver-agnostic: it asks ``resolve_chunk_size(execution_len)`` for the rows per
launch the runtime would use at that length (0 or ``None``: that length cannot run) and orders the candidates.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple, Union


def _ceil_to(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def default_chunk_resolver(max_rows: int, granule: int = 16) -> Callable[[int], int]:
    """Rows per launch of the packed-varlen prefill: the whole (16-row rounded) length up to ``max_rows`` per launch."""
    if max_rows < granule:
        raise ValueError(f"max_rows must be at least {granule}")
    cap = max_rows // granule * granule

    def resolve(execution_len: int) -> int:
        return min(_ceil_to(max(int(execution_len), 1), granule), cap)
    return resolve


def plan_bounded_prefill_execution(real_len: int, physical_limit: int, padding_budget: int,
                                   resolve_chunk_size: Callable[[int], Optional[int]], position: int = 0, *,
                                   alignment: int = 1, padding_rows: Union[str, int] = "auto",
                                   exact_chunk_size: Optional[int] = None,
                                   candidate_score: Optional[Callable[[int, int, int, int, int], tuple]] = None
                                   ) -> Tuple[int, int]:
    """``(execution_len, chunk_size)`` for appending ``real_len`` rows at ``position``.

    Candidates are the execution lengths ``ceil(real_len, alignment) + j * alignment`` with at most ``padding_budget``
    rows beyond the smallest aligned length (one exact length when ``padding_rows`` is an integer), that fit
    ``position + execution_len <= physical_limit``.  For each, ``resolve_chunk_size`` gives the rows per launch; a
    candidate is dropped when the resolver refuses it, when ``exact_chunk_size`` is given and differs, or when its last
    launch would contain padding only.  The winner minimises ``(launches, padding rows, tail deficit)`` - padding is
    chosen only when it saves a launch - or ``candidate_score(execution_len, chunk, launches, padding, tail_deficit)``
    when supplied.  Raises ``ValueError`` with the reason when nothing qualifies."""
    real_len, physical_limit, padding_budget = int(real_len), int(physical_limit), int(padding_budget)
    alignment, position = int(alignment), int(position)
    if real_len < 1:
        raise ValueError("prefill needs at least one real row")
    if alignment < 1 or padding_budget < 0 or position < 0:
        raise ValueError("alignment must be >= 1, padding_budget and position >= 0")
    if exact_chunk_size is not None:
        if isinstance(exact_chunk_size, bool) or not isinstance(exact_chunk_size, int) or exact_chunk_size <= 0 \
                or exact_chunk_size % 16:
            raise ValueError(f"exact_chunk_size must be a positive multiple of 16, got {exact_chunk_size!r}")
    room = physical_limit - position
    first = _ceil_to(real_len, alignment)
    if isinstance(padding_rows, str):
        if padding_rows != "auto":
            raise ValueError(f"padding_rows must be 'auto' or a non-negative integer, got {padding_rows!r}")
        lengths = range(first, first + padding_budget + 1, alignment)
    else:
        if isinstance(padding_rows, bool) or not isinstance(padding_rows, int) or padding_rows < 0:
            raise ValueError(f"padding_rows must be 'auto' or a non-negative integer, got {padding_rows!r}")
        exact = real_len + padding_rows
        if exact % alignment:
            raise ValueError(f"real_len + padding_rows = {exact} is not a multiple of the alignment {alignment}")
        lengths = (exact,)
    best, best_key, why = None, None, "no candidate length"
    for n_exec in lengths:
        if n_exec > room:
            why = f"position {position} + execution_len {n_exec} exceeds the physical limit {physical_limit}"
            break
        chunk = resolve_chunk_size(n_exec)
        if not chunk:
            why = f"the runtime has no chunk plan for execution_len {n_exec} at position {position}"
            continue
        chunk = int(chunk)
        if exact_chunk_size is not None and chunk != exact_chunk_size:
            why = f"execution_len {n_exec} resolves to chunk {chunk}, not the requested {exact_chunk_size}"
            continue
        launches = -(-n_exec // chunk)
        if (launches - 1) * chunk >= real_len:
            why = f"execution_len {n_exec} with chunk {chunk} would end in a launch of padding only"
            continue
        padding, deficit = n_exec - real_len, launches * chunk - n_exec
        key = candidate_score(n_exec, chunk, launches, padding, deficit) if candidate_score is not None \
            else (launches, padding, deficit)
        if best_key is None or key < best_key:
            best, best_key = (n_exec, chunk), key
    if best is None:
        raise ValueError(f"no bounded prefill plan for {real_len} rows at position {position}: {why}")
    return best


def chunk_policy_key(chunk_override: Union[int, str, None]) -> int:
    """What a handle's chunk policy contributes to its graph signatures: the explicit rows-per-launch override, 0 under
    ``"auto"`` (the resolved chunk is then a function of shape and resume position, which the signature already has)."""
    if chunk_override in (None, "auto", 0):
        return 0
    return int(chunk_override)


def prefill_position_key(seq_len: int, position: int) -> int:
    """Resume position of a multi-token forward for its graph signature.  Single-token steps return 0 so that every
    decode step shares one captured graph (position-dependent arguments live in device buffers that replay rereads);
    a prefill at position 0 also keys to 0."""
    return 0 if int(seq_len) <= 1 else int(position)


__all__ = ["plan_bounded_prefill_execution", "default_chunk_resolver", "chunk_policy_key", "prefill_position_key"]
