"""Summarise the steady-state part of a Chrome trace written by ``torch.profiler``.

The first steps of a run carry allocator growth, kernel loading and communicator set-up,
so only a window after them says anything about the steady state.  The window starts at
the ``--skip-steps``-th ``ProfilerStep#k`` range and covers ``--keep-steps`` of them (0 =
to the last one); a trace without such ranges falls back to skipping the first
``--fallback-skip-ratio`` of the time line.  Complete events (``ph == "X"``) that lie
entirely inside the window are summed by name; the share of communication is what
``nccl:`` / ``gloo:`` record_function ranges, NCCL device kernels and this library's fused
collective kernels account for.  Behaviour follows the reference's
``benchmarks/analyze_trace_stable_window.py`` (window rules ``:48-76``, summary
``:93-115``); added here: the fused-kernel names, a device-kernel-only share and
``--json``.

    python -m bitscom_b200.bench.trace_stable_window --trace trace.json --skip-steps 3
"""

from __future__ import annotations

import argparse
import json
from collections import defaultdict
from typing import Dict, Iterable, List, NamedTuple, Optional

COMM_PREFIXES = ("nccl:", "gloo:", "ncclDevKernel", "ncclKernel", "lowbit_collective",
                 "lowbit_emulated", "bitscom:")


class Window(NamedTuple):
    start_us: float
    end_us: float


def load_events(path: str) -> List[dict]:
    with open(path, encoding="utf-8") as f:
        data = json.load(f)
    return data["traceEvents"] if isinstance(data, dict) else data


def complete_events(events: Iterable[dict]) -> List[dict]:
    out = [e for e in events if e.get("ph") == "X" and "ts" in e and "dur" in e]
    out.sort(key=lambda e: e["ts"])
    return out


def profiler_steps(events: Iterable[dict]) -> List[dict]:
    return [e for e in complete_events(events)
            if isinstance(e.get("name"), str) and e["name"].startswith("ProfilerStep")]


def step_window(steps: List[dict], skip: int, keep: int) -> Window:
    if not steps:
        raise RuntimeError("no ProfilerStep ranges in the trace")
    if skip >= len(steps):
        raise RuntimeError(f"skip_steps={skip} leaves nothing of {len(steps)} profiler steps")
    last = len(steps) - 1 if keep <= 0 else min(len(steps) - 1, skip + keep - 1)
    return Window(float(steps[skip]["ts"]), float(steps[last]["ts"] + steps[last]["dur"]))


def time_window(ops: List[dict], skip_ratio: float) -> Window:
    if not ops:
        raise RuntimeError("no complete events in the trace")
    first = min(float(e["ts"]) for e in ops)
    last = max(float(e["ts"] + e["dur"]) for e in ops)
    span = max(last - first, 1.0)
    return Window(first + span * min(max(skip_ratio, 0.0), 0.95), last)


def events_in(events: Iterable[dict], w: Window) -> List[dict]:
    return [e for e in complete_events(events)
            if float(e["ts"]) >= w.start_us and float(e["ts"] + e["dur"]) <= w.end_us]


def is_comm(name) -> bool:
    return isinstance(name, str) and name.startswith(COMM_PREFIXES)


def summarize(events: List[dict], topk: int) -> Dict[str, object]:
    by_ms: Dict[str, float] = defaultdict(float)
    by_count: Dict[str, int] = defaultdict(int)
    kernel_ms = kernel_comm_ms = 0.0
    for e in events:
        name = e.get("name", "<unknown>")
        if isinstance(name, str) and name.startswith("ProfilerStep"):
            continue  # the step ranges are the ruler, not work
        ms = float(e["dur"]) / 1000.0
        by_ms[name] += ms
        by_count[name] += 1
        if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset"):
            kernel_ms += ms
            if is_comm(name):
                kernel_comm_ms += ms
    total = sum(by_ms.values())
    comm = sum(ms for n, ms in by_ms.items() if is_comm(n))
    top = sorted(by_ms.items(), key=lambda kv: -kv[1])[:topk]
    return {"events": sum(by_count.values()), "total_op_ms": total, "comm_op_ms": comm,
            "comm_share": comm / total if total > 0 else 0.0,
            "device_ms": kernel_ms, "device_comm_ms": kernel_comm_ms,
            "device_comm_share": kernel_comm_ms / kernel_ms if kernel_ms > 0 else 0.0,
            "top": [{"name": n, "ms": ms, "count": by_count[n]} for n, ms in top]}


def analyze(path: str, skip_steps: int = 3, keep_steps: int = 0, topk: int = 20,
            fallback_skip_ratio: float = 0.2) -> Dict[str, object]:
    events = load_events(path)
    steps = profiler_steps(events)
    window: Optional[Window]
    if steps:
        window, how = step_window(steps, skip_steps, keep_steps), "profiler_steps"
    else:
        window, how = time_window(complete_events(events), fallback_skip_ratio), "time_ratio"
    out = summarize(events_in(events, window), topk)
    out.update({"trace": path, "profiler_steps": len(steps), "window_by": how,
                "window_us": [window.start_us, window.end_us],
                "window_ms": (window.end_us - window.start_us) / 1000.0})
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="steady-state summary of a torch.profiler trace")
    ap.add_argument("--trace", required=True)
    ap.add_argument("--skip-steps", type=int, default=3,
                    help="initial ProfilerStep ranges to drop as warm-up")
    ap.add_argument("--keep-steps", type=int, default=0,
                    help="steps to keep after the warm-up (0 = all that remain)")
    ap.add_argument("--topk", type=int, default=20)
    ap.add_argument("--fallback-skip-ratio", type=float, default=0.2,
                    help="without ProfilerStep ranges, the leading fraction of time to drop")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    args = ap.parse_args(argv)
    r = analyze(args.trace, args.skip_steps, args.keep_steps, args.topk,
                args.fallback_skip_ratio)
    if args.json:
        print(json.dumps(r))
        return r
    print(f"trace: {r['trace']}")
    print(f"profiler steps found: {r['profiler_steps']}")
    if r["window_by"] == "time_ratio":
        print(f"no ProfilerStep found; time-based window, skip_ratio={args.fallback_skip_ratio}")
    print(f"stable window us: [{r['window_us'][0]:.0f}, {r['window_us'][1]:.0f}] "
          f"(duration {r['window_ms']:.3f} ms)")
    print(f"events in window: {r['events']}")
    print(f"window total op time: {r['total_op_ms']:.3f} ms")
    print(f"window comm op time: {r['comm_op_ms']:.3f} ms ({100 * r['comm_share']:.2f}%)")
    if r["device_ms"] > 0:
        print(f"device time: {r['device_ms']:.3f} ms, communication kernels "
              f"{r['device_comm_ms']:.3f} ms ({100 * r['device_comm_share']:.2f}%)")
    print("top ops by total ms:")
    for t in r["top"]:
        print(f"  {t['name']}: {t['ms']:.3f} ms, count={t['count']}")
    return r


if __name__ == "__main__":
    main()
