"""``python -m bitscom_b200 [info|build]``: what is built, what loads, which switches are set.

``info`` prints one JSON object: package and torch versions, the CUDA device if there is one,
for every native library whether its binary is present, up to date with the sources and
loadable, whether the ``lowbit`` backend extension imports, and the environment switches the
package reads.  ``build`` compiles everything in-tree (the same as ``setup.py build_ext``)."""

from __future__ import annotations

import json
import os
import sys

ENV_SWITCHES = [
    "BITSCOM_TIMING", "BITSCOM_TIMING_DIR", "BITSCOM_NVTX", "BITSCOM_COMM_DEBUG", "TRACE_EXPLAIN",
    "BITSCOM_UNSAFE_FULL_ASYNC_CHAIN", "BITSCOM_TIMEOUT_MS", "BITSCOM_MAX_CTAS", "BITSCOM_NVLS",
    "BITSCOM_LL_MAX_MB", "BITSCOM_SYMM_MB", "BITSCOM_GEMM",
    "BITSCOM_ATTN_FWD", "BITSCOM_ATTN_BWD_DQ", "BITSCOM_CPU_CODEC", "BITSCOM_ALLOW_FALLBACK",
    "BITSCOM_NO_BUILD", "BITSCOM_NVCC", "BITSCOM_CUDA_COMPILER", "BITSCOM_RUN_PERF",
    "BITSCOM_EXPERIMENTAL",
]


def info() -> dict:
    import torch

    import bitscom_b200
    from bitscom_b200 import _build

    libs = {}
    for name in _build.available_libraries():
        path = _build.lib_path(name)
        entry = {"path": path, "present": os.path.exists(path), "current": _build.is_current(name)}
        try:
            _build.load_library(name)
            entry["loads"] = True
        except Exception as exc:  # report, do not fail the report
            entry["loads"] = False
            entry["error"] = str(exc)[:200]
        libs[name] = entry
    out = {
        "package": bitscom_b200.__version__,
        "torch": torch.__version__,
        "cuda_available": torch.cuda.is_available(),
        "nvcc": _build.nvcc_path(),
        "libraries": libs,
        "backend_extension": bitscom_b200.is_extension_available(),
        "env": {k: os.environ[k] for k in ENV_SWITCHES if k in os.environ},
    }
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        out["device"] = {"name": p.name, "sm": f"{p.major}.{p.minor}",
                         "sms": p.multi_processor_count,
                         "memory_gb": round(p.total_memory / 2 ** 30, 1),
                         "count": torch.cuda.device_count()}
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    cmd = argv[0] if argv else "info"
    if cmd == "info":
        print(json.dumps(info(), indent=1))
        return 0
    if cmd == "build":
        from bitscom_b200 import _build, _ext

        for path in _build.build_all(force="-f" in argv):
            print("built", path)
        print("built", _ext.build_backend_extension())
        return 0
    print(__doc__)
    return 2


if __name__ == "__main__":
    sys.exit(main())
