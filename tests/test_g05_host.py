"""G0.5 adapter facade: entry points import, the action-expert profile guard names what differs, and every patch function
reports the missing runtime instead of falling back."""
from types import SimpleNamespace

import pytest


def _canonical_config(**over):
    from rpu_backend.adapters.g05 import CANONICAL
    rope = dict(rope_theta=CANONICAL.rope_theta, rope_type=CANONICAL.rope_type, mrope_section=list(CANONICAL.mrope_section),
                mrope_interleaved=CANONICAL.mrope_interleaved, partial_rotary_factor=CANONICAL.partial_rotary_factor)
    base = {k: getattr(CANONICAL, k) for k in CANONICAL.__dataclass_fields__ if k not in rope}
    base["layer_types"] = list(base["layer_types"])
    base.update(over)
    return SimpleNamespace(rope_parameters=rope, **base)


def test_profile_guard_accepts_canonical_and_names_differences():
    from rpu_backend.adapters import g05
    from rpu_backend.api.errors import UnsupportedModelError
    g05.check_action_profile(_canonical_config())
    assert g05.profile_mismatches(_canonical_config()) == []
    bad = _canonical_config(num_hidden_layers=12, input_dim=32)
    bad.rope_parameters["partial_rotary_factor"] = 1.0
    names = [m.split(":")[0] for m in g05.profile_mismatches(bad)]
    assert names == ["num_hidden_layers", "input_dim", "partial_rotary_factor"]
    with pytest.raises(UnsupportedModelError, match="num_hidden_layers: got 12"):
        g05.check_action_profile(bad)
    assert g05.SHARED_PREFIX_LAYERS == tuple(range(3, 24, 4))


def test_patch_entry_points_report_the_missing_runtime():
    from rpu_backend.adapters import g05
    from rpu_backend.api.errors import UnsupportedModelError
    for name in g05.__all__:
        if not name.startswith("patch_"):
            continue
        with pytest.raises(UnsupportedModelError, match="not built"):
            getattr(g05, name)(SimpleNamespace())
    # a wrong geometry is reported as a geometry problem, before the missing runtime
    with pytest.raises(UnsupportedModelError, match="head_dim: got 128"):
        g05.patch_g05_action_expert_for_rpu(SimpleNamespace(config=_canonical_config(head_dim=128)))
