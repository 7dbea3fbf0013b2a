"""CPU-only contracts of the vLLM integration: block tracking, release gate, plugin.

The scenarios are those the reference pins in ``tests/unit/test_open_blocks.py``
and ``tests/unit/test_vllm_compat.py``; vLLM itself is replaced by fake modules
injected at its import paths.
"""

from __future__ import annotations

import importlib
from importlib import metadata
import sys
from types import ModuleType, SimpleNamespace

import pytest

from fragpack_b200.integrations.vllm import capacity as cap
from fragpack_b200.integrations.vllm import compat
from fragpack_b200.integrations.vllm.lifecycle import OpenBlocks


def _so(new=(), cached=(), finished=(), resumed=(), preempted=(), updates=None):
    """Scheduler output with the fields OpenBlocks.update reads."""
    return SimpleNamespace(
        finished_req_ids=set(finished),
        preempted_req_ids=set(preempted),
        scheduled_new_reqs=[
            SimpleNamespace(req_id=r, block_ids=(list(b),), num_computed_tokens=c) for r, b, c in new
        ],
        block_table_updates={r: (ids,) for r, ids in updates.items()} if updates else None,
        scheduled_cached_reqs=SimpleNamespace(
            req_ids=[r for r, _, _ in cached],
            num_computed_tokens=[c for _, c, _ in cached],
            new_block_ids=[None if b is None else (list(b),) for _, _, b in cached],
            resumed_req_ids=set(resumed),
        ),
    )


def test_only_partially_written_blocks_are_live() -> None:
    t = OpenBlocks(128)
    t.update(_so(new=(("a", [10, 11, 12], 0), ("b", [20], 0))))
    assert t.live_blocks().tolist() == []
    t.update(_so(cached=(("a", 200, None), ("b", 128, None))))
    assert t.live_blocks().tolist() == [11]
    t.update(_so(cached=(("a", 300, None), ("b", 129, [21]))))
    assert sorted(t.live_blocks().tolist()) == [12, 21]


def test_finished_writer_frees_its_open_block_for_reuse() -> None:
    t = OpenBlocks(128)
    t.update(_so(new=(("a", [10, 11], 0),)))
    t.update(_so(cached=(("a", 200, None),)))
    t.update(_so(new=(("b", [30, 11], 0),), finished=("a",)))
    t.update(_so(cached=(("b", 50, None),)))
    assert t.live_blocks().tolist() == [30]


def test_resume_preempt_and_table_replacement() -> None:
    t = OpenBlocks(128)
    t.update(_so(new=(("a", [10, 11], 0),)))
    t.update(_so(cached=(("a", 150, None),)))
    t.update(_so(cached=(("a", 130, [40, 41]),), resumed=("a",)))
    assert t.live_blocks().tolist() == [41]
    # Preemption drops the request even if a stale cached row still names it.
    t.update(_so(preempted=("a",), cached=(("a", 160, None),)))
    assert t.live_blocks().tolist() == []
    # Preemption and re-admission in one step use the new allocation.
    t.update(_so(new=(("a", [10, 11], 150),)))
    t.update(_so(preempted=("a",), new=(("a", [50, 51], 130),)))
    assert t.live_blocks().tolist() == [51]
    # A full table replacement wins over the incremental list of the same step.
    t.update(_so(cached=(("a", 150, [90]),), updates={"a": [60, 61]}))
    assert t.live_blocks().tolist() == [61]
    t.update(_so(cached=(("a", 260, None),)))
    assert t.live_blocks().tolist() == []
    with pytest.raises(ValueError):
        OpenBlocks(0)


@pytest.fixture
def adapter(monkeypatch):
    module = importlib.reload(compat)
    monkeypatch.setattr(module.metadata, "version", lambda name: module.SUPPORTED_VLLM_VERSION)
    return module


def _fake_runner(monkeypatch) -> ModuleType:
    module = ModuleType("vllm.v1.worker.gpu.model_runner")

    class Runner:
        def execute_model(self, scheduler_output, *args, **kwargs):
            return scheduler_output, args, kwargs

    module.GPUModelRunner = Runner
    monkeypatch.setitem(sys.modules, module.__name__, module)
    return module


def _step():
    return _so(new=(("a", [10, 11], 150),))


@pytest.mark.parametrize("version", ["0.22.0", "0.30.0", "0.30.0+cu130", "0.31.0"])
def test_other_releases_are_rejected_before_patching(adapter, monkeypatch, version) -> None:
    runner = _fake_runner(monkeypatch)
    original = runner.GPUModelRunner.execute_model
    monkeypatch.setattr(adapter.metadata, "version", lambda name: version)
    with pytest.raises(RuntimeError, match="release-specific"):
        adapter.install_tracker(OpenBlocks(128), use_v2_model_runner=True)
    assert runner.GPUModelRunner.execute_model is original


def test_missing_vllm_and_v1_runner(adapter, monkeypatch) -> None:
    runner = _fake_runner(monkeypatch)
    original = runner.GPUModelRunner.execute_model
    with pytest.raises(ValueError, match="V2 model runner"):
        adapter.install_tracker(OpenBlocks(128), use_v2_model_runner=False)
    assert runner.GPUModelRunner.execute_model is original

    def missing(name):
        raise metadata.PackageNotFoundError(name)

    monkeypatch.setattr(adapter.metadata, "version", missing)
    with pytest.raises(RuntimeError, match="not installed"):
        adapter.require_supported_vllm()


def test_wrapper_tracks_real_steps_only_and_is_installed_once(adapter, monkeypatch) -> None:
    runner = _fake_runner(monkeypatch)
    tracker = OpenBlocks(128)
    inner = runner.GPUModelRunner.execute_model
    seen = []

    def observing(self, so, *args, **kwargs):
        seen.append(tracker.live_blocks().tolist())
        return inner(self, so, *args, **kwargs)

    runner.GPUModelRunner.execute_model = observing
    adapter.install_tracker(tracker, use_v2_model_runner=True)
    installed = runner.GPUModelRunner.execute_model
    step = _step()
    # The tracker is updated before the model runs, arguments pass through.
    assert runner.GPUModelRunner().execute_model(step, "x", flag=7) == (step, ("x",), {"flag": 7})
    assert seen == [[11]]
    # Dummy runs carry no scheduler metadata and leave the tracker alone.
    assert runner.GPUModelRunner().execute_model(None, dummy_run=True) == (None, (), {"dummy_run": True})
    assert tracker.live_blocks().tolist() == [11]
    adapter.install_tracker(tracker, use_v2_model_runner=True)
    assert runner.GPUModelRunner.execute_model is installed
    with pytest.raises(RuntimeError, match="already has a tracker"):
        adapter.install_tracker(OpenBlocks(128), use_v2_model_runner=True)


def test_plugin_registers_the_class_path_lazily(adapter, monkeypatch) -> None:
    from fragpack_b200.integrations.vllm import plugin

    registry = ModuleType("vllm.v1.attention.backends.registry")
    registry.AttentionBackendEnum = SimpleNamespace(CUSTOM="custom-slot")
    calls = []
    registry.register_backend = lambda slot, path: calls.append((slot, path))
    monkeypatch.setitem(sys.modules, registry.__name__, registry)
    backend = "fragpack_b200.integrations.vllm.backend"
    monkeypatch.setitem(sys.modules, backend, None)  # importing it would fail
    plugin.register()
    assert calls == [("custom-slot", backend + ".FragPackAttentionBackend")]
    monkeypatch.setattr(adapter.metadata, "version", lambda name: "0.31.0")
    with pytest.raises(RuntimeError, match="release-specific"):
        plugin.register()
    assert len(calls) == 1


def test_capacity_snapshot_is_published_and_copied() -> None:
    assert cap.get_capacity() is None or isinstance(cap.get_capacity(), cap.FragPackCapacity)
    snap = cap.FragPackCapacity(469, 128, 48, 4, 190464, 262144, {"arena": 1})
    cap.publish_capacity(snap)
    assert cap.get_capacity() is snap
    copy = snap.to_dict()
    copy["memory"]["arena"] = 2
    assert snap.memory["arena"] == 1
