"""In-tree build of the native libraries.

Every CUDA source under ``csrc/`` is compiled for sm_100a only with a direct ``nvcc``
call into ``bitscom_b200/lib/*.so`` and loaded with ``ctypes``: the kernels take raw
device pointers and a stream, so they need no torch headers and build in seconds.
The c10d backend (``_lowbit_c``) is the one torch C++ extension; it is built with
``torch.utils.cpp_extension`` into the same folder.

A library is rebuilt when the hash of its sources (and of the flags) changes.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from typing import Dict, List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIBDIR = os.path.join(_HERE, "lib")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
              "--expt-relaxed-constexpr"]

# library name -> (sources, extra flags)
LIBRARIES: Dict[str, dict] = {
    "bcom_codec": {"sources": ["codec_kernels.cu"], "deps": ["codec.cuh"], "flags": []},
    "bcom_comm": {"sources": ["fused_collectives.cu", "symm.cu"],
                  "deps": ["codec.cuh", "symm.h"], "flags": []},
    "bcom_cpu": {"sources": ["cpu_codec.cc"], "deps": [], "flags": [], "host_only": True},
    "bcom_llama": {"sources": ["gemm_tcgen05.cu", "attention_tcgen05.cu", "elementwise.cu"],
                   "deps": ["tc_common.cuh", "gemm_epilogue.cuh", "gemm_schedule.cuh", "no_alloc.h"],
                   "flags": []},
    # CTA-pair GEMM (opt-in variant): a library of its own, so that it can be left out of a
    # deployment without touching the default kernels
    "bcom_gemm2": {"sources": ["gemm_tcgen05_2cta.cu"],
                   "deps": ["tc_common.cuh", "gemm_epilogue.cuh", "gemm_schedule.cuh"],
                   "flags": []},
}

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def nvcc_path() -> Optional[str]:
    for cand in (os.environ.get("BITSCOM_NVCC"), os.environ.get("CUDA_NVCC_EXECUTABLE"),
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _existing(names: List[str]) -> List[str]:
    return [os.path.join(CSRC, n) for n in names if os.path.exists(os.path.join(CSRC, n))]


def _digest(name: str) -> str:
    spec = LIBRARIES[name]
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + spec["flags"]).encode())
    for path in _existing(spec["sources"]) + _existing(spec["deps"]):
        h.update(os.path.basename(path).encode())  # not the absolute path: the tree moves
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def lib_path(name: str) -> str:
    return os.path.join(LIBDIR, f"lib{name}.so")


def is_current(name: str) -> bool:
    so, stamp = lib_path(name), lib_path(name) + ".sha"
    if not (os.path.exists(so) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _digest(name)


def build_library(name: str, verbose: bool = False, force: bool = False) -> str:
    """Compile one library if its sources changed; returns the path of the .so."""
    spec = LIBRARIES[name]
    sources = _existing(spec["sources"])
    if not sources:
        raise FileNotFoundError(f"no sources for {name}")
    so = lib_path(name)
    if not force and is_current(name):
        return so
    os.makedirs(LIBDIR, exist_ok=True)
    if spec.get("host_only"):
        cxx = shutil.which("g++") or shutil.which("c++")
        if cxx is None:
            raise RuntimeError("g++ not found; cannot build " + name)
        # -ffp-contract=off: the codec must round every operation like the host quantizer
        cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-ffp-contract=off",
               "-fno-math-errno", "-fno-trapping-math", "-I", CSRC]
    else:
        nvcc = nvcc_path()
        if nvcc is None:
            raise RuntimeError("nvcc not found; cannot build " + name)
        cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + spec["flags"] + ["-I", CSRC]
        if verbose:
            cmd += ["-Xptxas", "-v"]
    tmp = f"{so}.{os.getpid()}.tmp"  # several ranks may build at once: private file, atomic rename
    cmd += ["-o", tmp] + sources
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"compiler failed for {name}:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    os.replace(tmp, so)
    stamp_tmp = f"{so}.sha.{os.getpid()}.tmp"
    with open(stamp_tmp, "w") as f:
        f.write(_digest(name))
    os.replace(stamp_tmp, so + ".sha")
    return so


def available_libraries() -> List[str]:
    return [n for n, spec in LIBRARIES.items() if _existing(spec["sources"])]


def build_all(verbose: bool = False, force: bool = False) -> List[str]:
    return [build_library(n, verbose=verbose, force=force) for n in available_libraries()]


def load_library(name: str) -> ctypes.CDLL:
    """dlopen a library, building it first when it is missing or stale and nvcc exists."""
    with _lock:
        if name in _loaded:
            return _loaded[name]
        so = lib_path(name)
        if not is_current(name):
            if nvcc_path() is not None or LIBRARIES[name].get("host_only"):
                build_library(name)
            elif not os.path.exists(so):
                raise RuntimeError(f"{so} is missing and nvcc is not available")
        lib = ctypes.CDLL(so, mode=ctypes.RTLD_GLOBAL)
        _loaded[name] = lib
        return lib


if __name__ == "__main__":
    for path in build_all(verbose="-v" in sys.argv, force="-f" in sys.argv):
        print("built", path)
