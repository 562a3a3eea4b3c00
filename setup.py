"""Packaging and the in-tree native build.

    python setup.py build_ext --inplace      # build every native library under bitscom_b200/lib
    pip install --no-build-isolation -e .    # editable install that does the same first

Unlike the reference's ``setup.py`` (two torch extensions compiled without ``-gencode``,
include / library discovery for several CUDA-like toolchains, ``setup.py:34-327``), there
is one target, sm_100a, and the CUDA libraries are plain shared objects built by direct
``nvcc`` calls (``bitscom_b200/_build.py``); only the c10d backend is a torch extension
(``bitscom_b200/_ext.py``).  Kept from the reference: the compiler can be chosen with
``BITSCOM_NVCC`` (the reference reads ``BITSCOM_CUDA_COMPILER``, honoured here as well),
and the build writes ``compile_commands.json`` at the repository root for clangd-style
tooling (the reference's ``BuildExtensionWithCompileCommands``, ``setup.py:235-287``).
"""

import json
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _version() -> str:
    with open(os.path.join(ROOT, "bitscom_b200", "__init__.py")) as f:
        for line in f:
            if line.startswith("__version__"):
                return line.split("=")[1].strip().strip("\"'")
    return "0.0.0"


def compile_commands() -> list:
    """One entry per native source with the command ``_build`` would run for it."""
    from bitscom_b200 import _build

    nvcc = _build.nvcc_path() or "nvcc"
    entries = []
    for name, spec in _build.LIBRARIES.items():
        for src in spec["sources"]:
            path = os.path.join(_build.CSRC, src)
            if not os.path.exists(path):
                continue
            if spec.get("host_only"):
                cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-pthread", "-ffp-contract=off",
                       "-I", _build.CSRC, "-c", path]
            else:
                cmd = [nvcc] + _build.ARCH_FLAGS + [f for f in _build.NVCC_FLAGS
                                                    if f != "-shared"] + \
                      spec["flags"] + ["-I", _build.CSRC, "-c", path]
            entries.append({"directory": ROOT, "file": path, "arguments": cmd})
    backend = os.path.join(_build.CSRC, "backend.cc")
    if os.path.exists(backend):
        try:
            from torch.utils import cpp_extension

            inc = [a for p in cpp_extension.include_paths("cuda") for a in ("-isystem", p)]
        except Exception:  # torch missing at packaging time: still list the file
            inc = []
        entries.append({"directory": ROOT, "file": backend,
                        "arguments": ["g++", "-O2", "-std=c++17", "-fPIC", "-DUSE_C10D_NCCL",
                                      "-DUSE_DISTRIBUTED", "-I", _build.CSRC] + inc +
                                     ["-c", backend]})
    return entries


class BuildNative(Command):
    """``build_ext``: compile the CUDA / C++ libraries and the c10d backend in-tree."""

    description = "build bitscom_b200's native libraries for sm_100a"
    user_options = [("inplace", "i", "accepted for familiarity; the build is always in-tree"),
                    ("force", "f", "rebuild even when the sources did not change"),
                    ("no-backend", None, "skip the torch c10d backend extension")]
    boolean_options = ["inplace", "force", "no-backend"]

    def initialize_options(self):
        self.inplace = False
        self.force = False
        self.no_backend = False

    def finalize_options(self):
        legacy = os.environ.get("BITSCOM_CUDA_COMPILER")
        if legacy and not os.environ.get("BITSCOM_NVCC"):
            os.environ["BITSCOM_NVCC"] = legacy

    def run(self):
        from bitscom_b200 import _build

        for path in _build.build_all(force=bool(self.force)):
            print("built", path)
        if not self.no_backend:
            try:
                from bitscom_b200 import _ext

                print("built", _ext.build_backend_extension())
            except ImportError as exc:  # no torch: the CUDA libraries alone still work
                print("skipped the c10d backend:", exc)
        out = os.path.join(ROOT, "compile_commands.json")
        with open(out, "w") as f:
            json.dump(compile_commands(), f, indent=1)
        print("wrote", out)


class BuildPyWithNative(build_py):
    def run(self):
        self.run_command("build_ext")
        super().run()


setup(
    name="bitscom_b200",
    version=_version(),
    description="Low-bit collectives for Blackwell: fused sm_100a kernels behind the bitscom API",
    packages=find_packages(include=["bitscom_b200", "bitscom_b200.*"]),
    package_data={"bitscom_b200": ["csrc/*", "lib/*.so"]},
    python_requires=">=3.10",
    entry_points={"console_scripts": ["bitscom-launch=bitscom_b200.launch:main",
                                      "bitscom-info=bitscom_b200.__main__:main"]},
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
)
