import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DETAIL mode wraps custom backends in a wrapper group that needs sequence numbers.
os.environ["TORCH_DISTRIBUTED_DEBUG"] = "OFF"

# where the reference's python/ folder is looked for: an explicit override, a checkout next to
# this repository, or the copy installed for the benchmark's reference arm
_REFERENCE_CANDIDATES = [
    os.environ.get("BITSCOM_REFERENCE_PYTHON"),
    os.path.join(os.path.dirname(ROOT), "reference", "python"),
    os.path.join(ROOT, "baseline", "_ref"),
]
REFERENCE_PYTHON = next(
    (c for c in _REFERENCE_CANDIDATES
     if c and os.path.exists(os.path.join(c, "bitscom", "quantization.py"))),
    _REFERENCE_CANDIDATES[1])


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")
    config.addinivalue_line("markers", "performance: timing comparisons")
    config.addinivalue_line("markers", "integration: end-to-end training loops")


@pytest.fixture(scope="session")
def reference_quantization():
    """The reference's pure-torch quantizer, used as the CPU oracle when it is mounted."""
    path = os.path.join(REFERENCE_PYTHON, "bitscom", "quantization.py")
    if not os.path.exists(path):
        pytest.skip("reference checkout not mounted")
    import importlib.util

    spec = importlib.util.spec_from_file_location("_reference_quantization", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["_reference_quantization"] = mod
    try:
        spec.loader.exec_module(mod)
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference quantizer not importable: {exc}")
    return mod
