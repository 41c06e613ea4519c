"""G0.5 (Galaxea, Qwen3.5 VLM + flow-matching action expert): the adapter's entry points and its profile guards.

The reference drives G0.5 by patching objects of the vendor's own Python package (policy, inferencer, data processor,
vision tower, VLM, action expert) so that their forwards run on its runtime.  That package is not part of this
environment, so the runtime halves are not built here; what is built is what does not need it:

* the eight ``patch_g05_*_for_rpu`` entry points, so that code written against the reference imports and gets a precise
  :class:`UnsupportedModelError` instead of an ``ImportError`` or a silent eager fallback;
* the action-expert profile guard: the one geometry the reference accepts, checked field by field with the offending
  fields named (``check_action_profile``), and the prefix layers the expert reads (``SHARED_PREFIX_LAYERS``: the
  full-attention layers of the 24-layer Qwen3.5 decoder, every fourth one).

The pieces such a runtime would be assembled from exist: the Qwen3.5 decoder with Gated DeltaNet layers and its vision
tower (``adapters/qwen3_5``), and an adaptive-norm action expert over prefix K/V with a graph-captured Euler loop
(``models/qwenpi05.py``; G0.5's expert differs in its M-RoPE sections, 25 % partial rotary, 27-D linear input / output
heads and adaLN conditioning).

Reference: ``python/rpu_backend/adapters/g05/__init__.py:1-25`` (facade), ``adapters/g05/action.py:12-56`` (profile),
``adapters/g05/runtime.py`` (patch functions).
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, List, Tuple

from ...api.errors import UnsupportedModelError

SHARED_PREFIX_LAYERS: Tuple[int, ...] = (3, 7, 11, 15, 19, 23)
ACTION_DIM_PAD = 32


@dataclass(frozen=True)
class G05ActionProfile:
    """The action-expert geometry of the published G0.5 checkpoint."""
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 8
    num_key_value_heads: int = 2
    head_dim: int = 256
    attention_bias: bool = False
    hidden_act: str = "silu"
    adaptive_mode: str = "adaLN"
    time_hidden_size: int = 1024
    input_type: str = "linear"
    input_dim: int = 27
    output_type: str = "linear"
    output_dim: int = 27
    use_final_norm: bool = True
    rms_norm_eps: float = 1.0e-6
    rope_theta: float = 10_000_000.0
    rope_type: str = "default"
    mrope_section: Tuple[int, ...] = (11, 11, 10)
    mrope_interleaved: bool = True
    partial_rotary_factor: float = 0.25
    layer_types: Tuple[str, ...] = ("full_attention",) * 24


CANONICAL = G05ActionProfile()
_ROPE_FIELDS = ("rope_theta", "rope_type", "mrope_section", "mrope_interleaved", "partial_rotary_factor")


def _read(config: Any, name: str):
    if name in _ROPE_FIELDS:
        rope = getattr(config, "rope_parameters", None) or {}
        return rope.get(name, getattr(config, name, None))
    return getattr(config, name, None)


def profile_mismatches(config: Any) -> List[str]:
    """``name: got X, the runtime takes Y`` for every field of ``config`` that differs from the canonical profile."""
    out = []
    for f in fields(G05ActionProfile):
        want, got = getattr(CANONICAL, f.name), _read(config, f.name)
        try:
            same = got is not None and type(want)(got) == want if not isinstance(want, tuple) else tuple(got) == want
        except (TypeError, ValueError):
            same = False
        if not same:
            out.append(f"{f.name}: got {got!r}, the runtime takes {want!r}")
    return out


def check_action_profile(config: Any) -> None:
    bad = profile_mismatches(config)
    if bad:
        raise UnsupportedModelError("G0.5 action expert: only the canonical Qwen3.5 action-expert profile is supported; "
                                    + "; ".join(bad))


def _needs_vendor_package(what: str):
    raise UnsupportedModelError(
        f"G0.5 {what}: the G0.5 runtime patches objects of the vendor's own Python package, which is not part of this "
        "build; the Qwen3.5 decoder / vision tower (adapters.qwen3_5) and the adaptive-norm action expert over prefix "
        "K/V (models.qwenpi05) are available as building blocks, the G0.5 assembly is not built")


def patch_g05_action_expert_for_rpu(expert, *args, **kwargs):
    """Checks the expert's profile first (a wrong geometry is reported as such), then reports the missing runtime."""
    cfg = getattr(expert, "config", None)
    if cfg is not None:
        check_action_profile(cfg)
    _needs_vendor_package("action expert")


def patch_g05_vlm_for_rpu(vlm, *args, **kwargs):
    _needs_vendor_package("VLM")


def patch_g05_vision_for_rpu(vision, *args, **kwargs):
    _needs_vendor_package("vision tower")


def patch_g05_policy_for_rpu(policy, *args, **kwargs):
    _needs_vendor_package("policy")


def patch_g05_inferencer_for_rpu(inferencer, *args, **kwargs):
    _needs_vendor_package("inferencer")


def patch_g05_data_processor_for_rpu(processor, *args, **kwargs):
    _needs_vendor_package("data processor")


def patch_g05_release_processor_for_rpu(processor, *args, **kwargs):
    _needs_vendor_package("release processor")


def patch_g05_release_runner_for_rpu(runner, *args, **kwargs):
    _needs_vendor_package("release runner")


__all__ = [
    "ACTION_DIM_PAD", "CANONICAL", "G05ActionProfile", "SHARED_PREFIX_LAYERS", "check_action_profile", "profile_mismatches",
    "patch_g05_action_expert_for_rpu", "patch_g05_data_processor_for_rpu", "patch_g05_inferencer_for_rpu",
    "patch_g05_policy_for_rpu", "patch_g05_release_processor_for_rpu", "patch_g05_release_runner_for_rpu",
    "patch_g05_vision_for_rpu", "patch_g05_vlm_for_rpu",
]
