import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand; nvcc cross-compiles without a GPU)."""
    from vllm_fp8_w8a16_sm70_b200 import _cabi, build
    build.build_library()
    return _cabi.load()


@pytest.fixture(scope="session")
def c_oracle():
    """oracle/c/libw8a16_ref.so, built on demand with gcc."""
    import ctypes
    import subprocess
    so = ROOT / "oracle" / "c" / "libw8a16_ref.so"
    src = ROOT / "oracle" / "c" / "w8a16_ref.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    return ctypes.CDLL(str(so))


@pytest.fixture(autouse=True)
def _device_healthy(request):
    """After every GPU test: no kernel may have recorded a timed-out wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from vllm_fp8_w8a16_sm70_b200 import ops
            st = ops.device_status(reset=True)
            if st != 0:
                ops.reset_workspaces()
            assert st == 0, f"device status word = {st:#x}: a kernel gave up on a bounded wait"
