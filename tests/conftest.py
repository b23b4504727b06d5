"""pytest configuration: the `gpu` marker and shared fixtures.

`-m "not gpu"` covers the oracle against numr's known answers, the host-side logic and
the C-ABI export surface; `-m gpu` holds the parity tests proper, which call the CUDA
path through the C ABI and compare it with the oracle.
"""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    O.lib()
    return O


@pytest.fixture(scope="session")
def nb_lib():
    """The C ABI, loaded (and built if missing)."""
    from numr_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def client():
    """A CudaClient on cuda:0 in exact-F32 mode; GPU tests fail loudly without a GPU."""
    import torch
    from numr_b200 import CudaClient
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return CudaClient(0, f32_mode="exact")


@pytest.fixture(scope="session")
def client_tf32():
    from numr_b200 import CudaClient
    return CudaClient(0, f32_mode="tf32")


@pytest.fixture
def tune(monkeypatch, nb_lib):
    """tune(NAME=value, ...) sets NUMR_B200_<NAME> switches and makes the library re-read them; the
    switches are removed (and re-read) when the test ends. A value of None removes a switch."""
    def apply(**switches):
        for name, value in switches.items():
            if value is None:
                monkeypatch.delenv("NUMR_B200_" + name, raising=False)
            else:
                monkeypatch.setenv("NUMR_B200_" + name, str(value))
        nb_lib.numr_b200_reload_tuning()
    yield apply
    monkeypatch.undo()
    nb_lib.numr_b200_reload_tuning()


@pytest.fixture(autouse=True)
def _check_kernel_status(request):
    """After every GPU test: no bounded wait may have run out."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import torch
        if torch.cuda.is_available():
            from numr_b200 import CudaClient
            st = CudaClient(0).device_status()
            assert st == 0, f"device status word is {st}: a bounded wait inside a kernel ran out"
