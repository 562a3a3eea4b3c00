"""setup.py: version, and the compile-command list covers every native source."""

import os
import subprocess
import sys

import bitscom_b200
from bitscom_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_setup_reports_package_version():
    out = subprocess.run([sys.executable, "setup.py", "--version"], cwd=ROOT,
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip().splitlines()[-1] == bitscom_b200.__version__


def test_compile_commands_cover_all_sources():
    code = ("import sys, json; sys.argv=['setup.py','--version']; "
            "ns={'__name__':'setup_probe','__file__':'setup.py'}; "
            "src=open('setup.py').read().split('\\nsetup(\\n')[0]; exec(compile(src,'setup.py','exec'),ns); "
            "print(json.dumps([e['file'] for e in ns['compile_commands']()]))")
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json

    files = {os.path.basename(f) for f in json.loads(out.stdout.strip().splitlines()[-1])}
    want = {s for spec in _build.LIBRARIES.values() for s in spec["sources"]} | {"backend.cc"}
    assert want <= files


def test_c_host_example_links_against_the_cpu_codec(tmp_path):
    """The C API is callable from a plain C program (examples/cpu_codec_example.c)."""
    import shutil

    import pytest

    from bitscom_b200.ops import cpu_codec

    cc = shutil.which("cc") or shutil.which("gcc")
    if cc is None or not cpu_codec.available():
        pytest.skip("needs a C compiler and the CPU codec library")
    libdir = os.path.dirname(_build.lib_path("bcom_cpu"))
    exe = str(tmp_path / "example")
    build = subprocess.run([cc, os.path.join(ROOT, "examples", "cpu_codec_example.c"),
                            f"-L{libdir}", "-lbcom_cpu", "-lm", f"-Wl,-rpath,{libdir}", "-o", exe],
                           capture_output=True, text=True, timeout=120)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "packed bytes" in run.stdout


def test_info_command_reports_libraries():
    out = subprocess.run([sys.executable, "-m", "bitscom_b200", "info"], cwd=ROOT,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json

    rep = json.loads(out.stdout)
    assert rep["package"] == bitscom_b200.__version__
    assert set(rep["libraries"]) == set(_build.available_libraries())
    assert rep["libraries"]["bcom_cpu"]["loads"] is True
    bad = subprocess.run([sys.executable, "-m", "bitscom_b200", "bogus"], cwd=ROOT,
                         capture_output=True, text=True, timeout=120)
    assert bad.returncode == 2
