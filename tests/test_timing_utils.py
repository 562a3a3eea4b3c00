"""Timing / logging utilities: the log is off by default (the reference writes it on every
call), counters accumulate, spans show up as profiler ranges."""

import os

import torch

from bitscom_b200.utils import timing


def test_log_is_off_by_default_and_opt_in(tmp_path, monkeypatch):
    monkeypatch.delenv("BITSCOM_TIMING", raising=False)
    monkeypatch.setenv("BITSCOM_TIMING_DIR", str(tmp_path))
    timing.log("nothing should be written")
    with timing.span("quiet"):
        pass
    assert os.listdir(tmp_path) == []
    monkeypatch.setenv("BITSCOM_TIMING", "1")
    with timing.span("phase_one"):
        pass
    timing.log("hello")
    files = os.listdir(tmp_path)
    assert files == ["bitscom_rank-1.log"]            # no process group: rank -1
    text = (tmp_path / files[0]).read_text()
    assert "phase_one elapsed_ms=" in text and "hello" in text


def test_counters_accumulate_and_reset():
    timing.reset_counters()
    timing.add("buckets")
    timing.add("buckets")
    timing.add("bytes", 1024)
    assert timing.counters() == {"buckets": 2.0, "bytes": 1024.0}
    snapshot = timing.counters()
    snapshot["buckets"] = 99                          # a copy, not the live table
    assert timing.counters()["buckets"] == 2.0
    timing.reset_counters()
    assert timing.counters() == {}


def test_span_is_a_profiler_range():
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        with timing.span("inside"):
            torch.ones(8).sum()
    assert any(e.name == "bitscom:inside" for e in prof.events())
