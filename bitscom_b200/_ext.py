"""Build / load the one torch C++ extension: the ``lowbit`` c10d backend
(``csrc/backend.cc`` -> ``bitscom_b200/lib/_lowbit_c.so``), linked against the fused
collectives library ``libbcom_comm.so`` in the same folder."""

from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

from . import _build

NAME = "_lowbit_c"
SOURCE = os.path.join(_build.CSRC, "backend.cc")
DEPS = [os.path.join(_build.CSRC, "symm.h")]


def _so_path() -> str:
    return os.path.join(_build.LIBDIR, NAME + ".so")


def _digest() -> str:
    h = hashlib.sha256()
    for path in [SOURCE] + DEPS:
        with open(path, "rb") as f:
            h.update(f.read())
    import torch

    h.update(torch.__version__.encode())
    return h.hexdigest()


def _current() -> bool:
    so, stamp = _so_path(), _so_path() + ".sha"
    if not (os.path.exists(so) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _digest()


def build_backend_extension(verbose: bool = False) -> str:
    """Compile the backend if its sources changed; returns the path of the module."""
    if _current():
        return _so_path()
    from torch.utils import cpp_extension

    _build.build_library("bcom_comm")
    build_dir = os.path.join(_build.LIBDIR, f"_build_{NAME}_{os.getpid()}")
    os.makedirs(build_dir, exist_ok=True)
    nccl_inc = []
    for base in sys.path:
        cand = os.path.join(base, "nvidia", "nccl", "include")
        if os.path.exists(os.path.join(cand, "nccl.h")):
            nccl_inc.append(cand)
            break
    cpp_extension.load(
        name=NAME, sources=[SOURCE], build_directory=build_dir, verbose=verbose,
        extra_cflags=["-O2", "-std=c++17", "-DUSE_C10D_NCCL", "-DUSE_DISTRIBUTED"],
        extra_include_paths=[_build.CSRC] + nccl_inc + cpp_extension.include_paths("cuda"),
        extra_ldflags=[f"-L{_build.LIBDIR}", "-lbcom_comm", "-Wl,-rpath,$ORIGIN",
                       "-Wl,-rpath," + _build.LIBDIR],
        with_cuda=True, is_python_module=False)
    built = os.path.join(build_dir, NAME + ".so")
    os.replace(built, _so_path())
    stamp_tmp = f"{_so_path()}.sha.{os.getpid()}.tmp"
    with open(stamp_tmp, "w") as f:
        f.write(_digest())
    os.replace(stamp_tmp, _so_path() + ".sha")
    return _so_path()


def load_backend_extension():
    """Import the backend module, building it when nvcc/g++ are present and it is stale."""
    import torch  # noqa: F401  (registers the c10d pybind types the module derives from)
    import torch.distributed  # noqa: F401

    so = _so_path()
    if not _current():
        if os.environ.get("BITSCOM_NO_BUILD", "0") == "1" and os.path.exists(so):
            pass
        else:
            so = build_backend_extension()
    _build.load_library("bcom_comm")
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
