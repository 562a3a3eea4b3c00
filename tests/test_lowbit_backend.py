"""Backend registration and option resolution (reference tests/test_lowbit_backend.py)."""

import pytest

import bitscom_b200.lowbit_backend as lb


@pytest.fixture
def fresh(monkeypatch):
    registered = {}

    def register_backend(name, func, devices=None, **kw):
        registered.update(name=name, func=func, devices=devices)

    created = {}

    def create_backend(**kwargs):
        created.update(kwargs)
        return "pg"

    monkeypatch.setattr(lb.dist.Backend, "register_backend", register_backend)
    monkeypatch.setattr(lb, "_REGISTERED", False)
    monkeypatch.setattr(lb, "_HAS_EXTENSION", True)
    monkeypatch.setattr(lb, "_EXTENSION_IMPORT_ERROR", None)
    monkeypatch.setattr(lb, "create_backend", create_backend)
    for name, val in (("_BACKEND_BITWIDTH", 4), ("_BACKEND_ERROR_FEEDBACK", False),
                      ("_BACKEND_ERROR_FEEDBACK_MODE", "none"), ("_BACKEND_BLOCK_SIZE", 256),
                      ("_BACKEND_STAGE2_ERROR_FEEDBACK", False)):
        monkeypatch.setattr(lb, name, val)
    return registered, created


def test_register_records_options(fresh):
    registered, _ = fresh
    lb.register_lowbit_backend(bitwidth=2, error_feedback=True, block_size=128)
    assert registered["name"] == "lowbit" and registered["devices"] == ["cpu", "cuda"]
    assert (lb._BACKEND_BITWIDTH, lb._BACKEND_ERROR_FEEDBACK, lb._BACKEND_ERROR_FEEDBACK_MODE,
            lb._BACKEND_BLOCK_SIZE, lb._BACKEND_STAGE2_ERROR_FEEDBACK) == (
        2, True, "legacy", 128, False)


def test_register_is_idempotent_and_conflicts_raise(fresh):
    lb.register_lowbit_backend(bitwidth=4, error_feedback_mode="ef21+")
    assert lb._BACKEND_ERROR_FEEDBACK_MODE == "ef21_plus"
    assert lb._BACKEND_STAGE2_ERROR_FEEDBACK is True
    lb.register_lowbit_backend(bitwidth=4, error_feedback_mode="ef21_plus")
    with pytest.raises(RuntimeError, match="already registered with different options"):
        lb.register_lowbit_backend(bitwidth=2)


def test_mode_aliases_and_validation(fresh):
    assert lb.resolve_options(4, False, "ef", 256, None) == (4, True, "legacy", 256, False)
    assert lb.resolve_options(4, True, "auto", 256, None)[2] == "legacy"
    assert lb.resolve_options(4, True, "none", 256, None)[1] is False
    assert lb.resolve_options(4, False, "ef21", 256, True)[4] is True
    with pytest.raises(ValueError):
        lb.resolve_options(4, False, "bogus", 256, None)
    with pytest.raises(ValueError):
        lb.resolve_options(3, False, None, 256, None)
    with pytest.raises(ValueError):
        lb.resolve_options(4, False, None, 0, None)


def test_missing_extension_raises(fresh, monkeypatch):
    monkeypatch.setattr(lb, "_HAS_EXTENSION", False)
    with pytest.raises(RuntimeError, match="extension is not available"):
        lb.register_lowbit_backend()
    with pytest.raises(RuntimeError, match="extension is not available"):
        lb._create_lowbit_pg(None, 0, 1, None)


def test_factory_passes_options(fresh):
    _, created = fresh
    lb.register_lowbit_backend(bitwidth=1, error_feedback_mode="ef21_plus", block_size=64,
                               stage2_error_feedback=False)
    assert lb._create_lowbit_pg("store", 3, 8, "timeout") == "pg"
    assert created == dict(store="store", rank=3, size=8, timeout="timeout", bitwidth=1,
                           error_feedback=True, error_feedback_mode="ef21_plus",
                           block_size=64, stage2_error_feedback=False)
