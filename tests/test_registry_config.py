import pytest

from elf_b200 import PipelineConfig, Placement
from elf_b200.registry import COMM_SCHEDULERS, PARTITIONERS, SCHEDULERS, TRACERS, Registry, resolve
import elf_b200.partitioners  # noqa: F401  (registers partitioners and tracers)


def test_default_config():
    cfg = PipelineConfig()
    assert cfg.tracer == "default" and cfg.partitioner == "constrained" and cfg.scheduler == "auto"
    assert cfg.comm_scheduler == "pipelined" and cfg.placement == "auto"
    assert cfg.pp is None and cfg.dp == 1 and cfg.worker == 0 and cfg.memory_budget is None and cfg.signatures is None


def test_custom_config_and_kwargs():
    cfg = PipelineConfig(scheduler="zbh2", dp=2, pp=4, memory_budget=1000, partitioner=False)
    kw = cfg.to_kwargs()
    assert kw["scheduler"] == "zbh2" and kw["dp"] == 2 and kw["pp"] == 4 and kw["memory_budget"] == 1000
    assert "signatures" not in kw and kw["partitioner"] is False
    r = cfg.resolve()
    assert r.scheduler is SCHEDULERS["zbh2"] and r.partitioner is False and callable(r.comm_scheduler)


def test_registry_contents():
    for k in ["afab", "gpipe", "1f1b", "megatron", "hanayo", "full_remat", "zbh1", "zbh2", "zbv", "inference", "fixed", "auto"]:
        assert k in SCHEDULERS
    assert sorted(PARTITIONERS.available()) == ["constrained", "dagP", "metis", "naive"]
    assert sorted(TRACERS.available()) == ["default", "export", "fx", "fx_safe"]
    assert sorted(COMM_SCHEDULERS.available()) == ["pipelined", "simulation", "topo"]
    assert SCHEDULERS.get_key(SCHEDULERS["gpipe"]) == "afab"
    assert "afab" in SCHEDULERS.available() and "gpipe" not in SCHEDULERS.available()


def test_registry_api():
    reg = Registry("thing")
    f = lambda: 1
    assert reg.register(["a", "b"], f, "desc") is f
    assert reg["a"] is f and reg.get("b") is f and len(reg) == 2 and list(reg) == ["a", "b"]
    assert reg.get_description("b") == "desc" and reg.available() == ["a"]
    with pytest.raises(KeyError):
        reg.register("a", lambda: 2)
    with pytest.raises(KeyError):
        reg.get("zzz")
    with pytest.raises(ValueError):
        reg.get_key(object())
    assert resolve(f, reg) is f and resolve("a", reg) is f
    with pytest.raises(ValueError, match="Available"):
        resolve("nope", reg)


def test_auto_scheduler_needs_a_budget():
    with pytest.raises(RuntimeError, match="memory_budget"):
        SCHEDULERS["auto"]([0, 1], 4)


def test_placement():
    assert list(Placement.default("zbv", 4)) == [0, 1, 2, 3, 3, 2, 1, 0]
    assert list(Placement.default("hanayo", 2)) == [0, 1, 1, 0]
    assert list(Placement.default("megatron", 2)) == [0, 1, 0, 1]
    assert list(Placement.default("1f1b", 3)) == [0, 1, 2]
    assert list(Placement.default(lambda p, n: [], 2)) == [0, 1]
    p = Placement([0, 1, 1, 2])
    assert p.get_ids(1) == [1, 2] and p.head() == 0 and p.tail() == 2 and p.is_head(0) and p.is_tail(2)
    assert list(p.add_offset(4)) == [4, 5, 5, 6] and list(p.add_offset(4).normalised()) == [0, 1, 1, 2]
    assert isinstance(Placement([0, 1]) * 2, Placement) and list(Placement([0, 1]) * 2) == [0, 1, 0, 1]
