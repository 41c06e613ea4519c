"""RhinoVLAPolicy: lifecycle and execution handshake, driven with fake runtimes on the host."""
import pathlib
import sys
import types

import pytest

from rhinoforge_b200.api import RhinoVLAPolicy, UnsupportedModelError
from rhinoforge_b200.api._unbuilt import unbuilt_facade
from rhinoforge_b200.api.rhinovla import StagePlan, declared_capabilities, resolve_runtime_factory

CAPS = {"prefill": ("chunk_size", "padding_rows", "padding_budget"), "action": ("chunk_size",)}


class FakeRuntime:
    """Publishes a resolved plan per dispatch the way a real runtime has to."""

    _rpu_execution_capabilities = CAPS

    def __init__(self, config=None, rpu_execution=None, *, logical=100, align=None, publish=True, chunk=None, pad=None):
        self.config = config
        if rpu_execution is not None:
            self._rpu_execution = rpu_execution
        self._logical, self._align, self._publish, self._chunk, self._pad = logical, align, publish, chunk, pad
        self._rpu_execution_resolved_generation = 0
        self.calls = []

    def _resolve(self):
        if not self._publish:
            return
        req = dict(getattr(self, "_rpu_execution", {}).get("prefill", {}))
        chunk = self._chunk or (req.get("chunk_size") if isinstance(req.get("chunk_size"), int) else 256)
        pad = self._pad if self._pad is not None else (
            req["padding_rows"] if isinstance(req.get("padding_rows"), int) else (-self._logical) % (self._align or 1))
        plan = {"logical_len": self._logical, "execution_len": self._logical + pad, "chunk_size": chunk,
                "padding_rows": pad}
        if self._align:
            plan["execution_alignment"] = self._align
        self._rpu_execution_resolved = {"prefill": plan, "action": {"logical_len": 50, "execution_len": 50,
                                                                      "chunk_size": 64, "padding_rows": 0}}
        self._rpu_execution_resolved_generation += 1

    def prepare_graphs(self, **request):
        self.calls.append(("prepare", request))
        self._resolve()
        return "prepared"

    def predict(self, **request):
        self.calls.append(("predict", request))
        self._resolve()
        return {"actions": [0.0] * 7}


def test_constructor_is_closed_and_other_families_still_refuse():
    with pytest.raises(RuntimeError, match="not a public constructor"):
        RhinoVLAPolicy()
    Stub = unbuilt_facade("SomePolicy", "some family", "needs its runtime")
    with pytest.raises(UnsupportedModelError, match="some family"):
        Stub.from_pretrained("x")
    with pytest.raises(UnsupportedModelError):
        Stub()


def test_from_runtime_without_execution_config_is_a_plain_wrapper():
    rt = FakeRuntime()
    pol = RhinoVLAPolicy.from_runtime(rt)
    assert pol.runtime is rt and not pol.rpu_execution and pol.last_rpu_execution_plan == {}
    assert pol.predict(image=1)["actions"] and pol.predict_action_chunk(image=2)["actions"]
    assert pol.prepare_graphs(image=0) == "prepared"
    assert [c[0] for c in rt.calls] == ["predict", "predict", "prepare"]
    assert pol.last_rpu_execution_plan == {}                        # no handshake was asked for
    assert RhinoVLAPolicy.from_runtime(pol) is pol
    with pytest.raises(TypeError, match="predict"):
        RhinoVLAPolicy.from_runtime(object())


def test_from_runtime_adopts_the_runtimes_own_configuration():
    rt = FakeRuntime(rpu_execution={"prefill": {"chunk_size": 128}})
    pol = RhinoVLAPolicy.from_runtime(rt)
    assert pol.rpu_execution == {"prefill": {"chunk_size": 128}}
    pol.predict()
    assert pol.last_rpu_execution_plan == {}                        # adopted, not requested: nothing to verify
    with pytest.raises(ValueError, match="conflicts"):
        RhinoVLAPolicy.from_runtime(rt, rpu_execution={"prefill": {"chunk_size": 256}})
    with pytest.raises(ValueError, match="existing policy"):
        RhinoVLAPolicy.from_runtime(pol, rpu_execution={"prefill": {"chunk_size": 256}})
    same = RhinoVLAPolicy.from_runtime(pol, rpu_execution={"prefill": {"chunk_size": 128}})
    assert same is pol
    pol.predict()
    assert pol.last_rpu_execution_plan["prefill"]["chunk_size"] == 128   # re-wrapping with a request turns it on


def test_a_request_the_runtime_never_saw_is_refused():
    with pytest.raises(ValueError, match="not consumed"):
        RhinoVLAPolicy.from_runtime(FakeRuntime(), rpu_execution={"prefill": {"chunk_size": 128}})
    bare = types.SimpleNamespace(predict=lambda **kw: None)
    with pytest.raises(ValueError, match="_rpu_execution_capabilities"):
        RhinoVLAPolicy.from_runtime(bare, rpu_execution={"prefill": {"chunk_size": 128}})
    assert RhinoVLAPolicy.from_runtime(bare, rpu_execution={}).rpu_execution == {}


def test_from_factory_passes_config_and_validates_the_plan():
    seen = {}

    def factory(config, rpu_execution=None):
        seen["config"], seen["exec"] = config, rpu_execution
        return FakeRuntime(config, rpu_execution, logical=100, align=16)
    factory._rpu_execution_capabilities = CAPS

    pol = RhinoVLAPolicy.from_factory(factory, {"ckpt": "x"}, rpu_execution={"prefill": {"chunk_size": 128,
                                                                                         "padding_budget": 0}})
    assert seen["config"] == {"ckpt": "x"} and seen["exec"]["prefill"]["chunk_size"] == 128
    with pytest.raises(TypeError):
        seen["exec"]["prefill"]["chunk_size"] = 1                   # frozen before it reaches the factory
    pol.predict(prompt="pick")
    plan = pol.last_rpu_execution_plan
    assert plan == {"prefill": {"logical_len": 100, "execution_len": 112, "chunk_size": 128, "padding_rows": 12,
                                "execution_alignment": 16}}
    plan["prefill"]["chunk_size"] = 0
    assert pol.last_rpu_execution_plan["prefill"]["chunk_size"] == 128  # the property hands out copies
    # without rpu_execution the factory is called with the config alone
    RhinoVLAPolicy.from_factory(lambda config: FakeRuntime(config), {"a": 1})
    with pytest.raises(TypeError, match="mapping"):
        RhinoVLAPolicy.from_factory(factory, ["not", "a", "mapping"])


def test_capabilities_gate_the_request_before_the_factory_runs():
    ran = []

    def factory(config, rpu_execution=None):
        ran.append(1)
        return FakeRuntime(config, rpu_execution)
    factory._rpu_execution_capabilities = {"action": ("chunk_size",)}
    with pytest.raises(ValueError, match="not supported"):
        RhinoVLAPolicy.from_factory(factory, {}, rpu_execution={"prefill": {"chunk_size": 128}})
    with pytest.raises(ValueError, match="not supported"):
        RhinoVLAPolicy.from_factory(factory, {}, rpu_execution={"action": {"padding_rows": 0}})
    with pytest.raises(ValueError, match="unknown stage"):
        RhinoVLAPolicy.from_factory(factory, {}, rpu_execution={"decode": {}})
    assert not ran
    for bad, exc in (({"bogus": ()}, ValueError), ({"action": "chunk_size"}, TypeError),
                     ({"action": ("rows",)}, ValueError), (["action"], TypeError)):
        with pytest.raises(exc):
            declared_capabilities(types.SimpleNamespace(_rpu_execution_capabilities=bad), "t")
    assert declared_capabilities(types.SimpleNamespace(
        _rpu_execution_capabilities={"prefill": {"padding_budget", "chunk_size"}}), "t") == {
            "prefill": ("chunk_size", "padding_budget")}


@pytest.mark.parametrize("kwargs, request_cfg, message", [
    (dict(publish=False), {"prefill": {"chunk_size": 128}}, "fresh resolved execution plan"),
    (dict(chunk=256), {"prefill": {"chunk_size": 128}}, "does not match exact request 128"),
    (dict(pad=4), {"prefill": {"padding_rows": 0}}, "padding_rows=4 does not match"),
    (dict(align=16, pad=28), {"prefill": {"padding_budget": 8}}, "exceeds budget 8"),
    (dict(chunk=100), {"prefill": {"chunk_size": "auto"}}, "invalid resolved 'prefill' plan"),
    (dict(align=16, pad=3), {"prefill": {"chunk_size": "auto"}}, "invalid resolved 'prefill' plan"),
])
def test_a_runtime_that_ignores_the_request_is_caught(kwargs, request_cfg, message):
    def factory(config, rpu_execution=None):
        return FakeRuntime(config, rpu_execution, **kwargs)
    factory._rpu_execution_capabilities = CAPS
    pol = RhinoVLAPolicy.from_factory(factory, {}, rpu_execution=request_cfg)
    with pytest.raises(RuntimeError, match=message):
        pol.predict()
    assert pol.last_rpu_execution_plan == {}


def test_mandatory_alignment_padding_does_not_count_against_the_budget():
    def factory(config, rpu_execution=None):
        return FakeRuntime(config, rpu_execution, logical=100, align=16, pad=12 + 16)
    factory._rpu_execution_capabilities = CAPS
    pol = RhinoVLAPolicy.from_factory(factory, {}, rpu_execution={"prefill": {"padding_budget": 16}})
    assert pol.prepare_graphs() == "prepared"
    assert pol.last_rpu_execution_plan["prefill"]["padding_rows"] == 28


def test_stage_plan_parsing():
    ok = {"logical_len": 10, "execution_len": 16, "chunk_size": 32, "padding_rows": 6}
    p = StagePlan.parse("vision", ok, "t")
    assert p.alignment == 1 and p.mandatory_padding == 0 and p.as_dict() == ok
    with pytest.raises(RuntimeError, match="missing stage"):
        StagePlan.parse("vision", None, "t")
    with pytest.raises(RuntimeError, match=r"missing=\['chunk_size'\]"):
        StagePlan.parse("vision", {k: v for k, v in ok.items() if k != "chunk_size"}, "t")
    with pytest.raises(RuntimeError, match=r"unknown=\['extra'\]"):
        StagePlan.parse("vision", {**ok, "extra": 1}, "t")
    with pytest.raises(TypeError, match="integers"):
        StagePlan.parse("vision", {**ok, "chunk_size": True}, "t")
    with pytest.raises(RuntimeError, match="invalid"):
        StagePlan.parse("vision", {**ok, "execution_len": 17}, "t")
    with pytest.raises(RuntimeError, match="invalid"):
        StagePlan.parse("vision", {**ok, "execution_alignment": 0}, "t")


def test_generation_counter_must_be_a_real_integer():
    rt = FakeRuntime(rpu_execution={"prefill": {"chunk_size": 128}})
    pol = RhinoVLAPolicy.from_runtime(rt, rpu_execution={"prefill": {"chunk_size": 128}})
    rt._rpu_execution_resolved_generation = True
    with pytest.raises(TypeError, match="non-negative integer"):
        pol.predict()
    rt._rpu_execution_resolved_generation = 3
    pol.predict()
    assert rt._rpu_execution_resolved_generation == 4 and pol.last_rpu_execution_plan


def test_a_failing_predict_propagates_and_keeps_the_previous_plan():
    rt = FakeRuntime(rpu_execution={"prefill": {"chunk_size": 128}})
    pol = RhinoVLAPolicy.from_runtime(rt, rpu_execution={"prefill": {"chunk_size": 128}})
    pol.predict()
    before = pol.last_rpu_execution_plan

    def boom(**kw):
        raise KeyError("camera")
    rt.predict = boom
    with pytest.raises(KeyError):
        pol.predict()
    assert pol.last_rpu_execution_plan == before
    rt.prepare_graphs = None                                        # present but not callable
    with pytest.raises(TypeError, match="prepare_graphs"):
        pol.prepare_graphs()


def test_from_pretrained_forwards_path_config_and_kwargs(tmp_path, monkeypatch):
    mod = types.ModuleType("fake_rhinovla_repo")
    got = {}

    def build_runtime(path, **kw):
        got["path"], got["kw"] = path, kw
        return FakeRuntime(kw.get("config"), kw.get("rpu_execution"))
    build_runtime._rpu_execution_capabilities = CAPS
    mod.build_runtime, mod.not_callable = build_runtime, 3
    monkeypatch.setitem(sys.modules, "fake_rhinovla_repo", mod)

    pol = RhinoVLAPolicy.from_pretrained(tmp_path, runtime_factory="fake_rhinovla_repo:build_runtime",
                                         config={"views": 3}, rpu_execution={"action": {"chunk_size": 64}}, device="cuda:0")
    assert got["path"] == tmp_path and isinstance(got["path"], pathlib.Path)
    assert got["kw"]["config"] == {"views": 3} and got["kw"]["device"] == "cuda:0"
    assert got["kw"]["rpu_execution"] == {"action": {"chunk_size": 64}}
    pol.predict()
    assert pol.last_rpu_execution_plan == {"action": {"logical_len": 50, "execution_len": 50, "chunk_size": 64,
                                                      "padding_rows": 0}}
    RhinoVLAPolicy.from_pretrained("repo/name", runtime_factory=build_runtime)
    assert got["kw"] == {}
    with pytest.raises(ValueError, match="must not be empty"):
        RhinoVLAPolicy.from_pretrained("", runtime_factory=build_runtime)
    with pytest.raises(TypeError, match="str or PathLike"):
        RhinoVLAPolicy.from_pretrained(7, runtime_factory=build_runtime)
    with pytest.raises(TypeError, match="must be a mapping"):
        RhinoVLAPolicy.from_pretrained("x", runtime_factory=build_runtime, config=[1])
    with pytest.raises(ValueError, match="module:callable"):
        resolve_runtime_factory("fake_rhinovla_repo.build_runtime")
    with pytest.raises(TypeError, match="not callable"):
        resolve_runtime_factory("fake_rhinovla_repo:not_callable")
    with pytest.raises(TypeError, match="callable or"):
        resolve_runtime_factory(12)
