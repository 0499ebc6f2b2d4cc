import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """The package directory name has a hyphen, so it is loaded by path."""
    name = "llm_sys_project_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg = os.path.join(ROOT, "llm-sys-project_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg, "__init__.py"),
                                                  submodule_search_locations=[pkg])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def b200():
    return load_package()


@pytest.fixture(scope="session")
def cuda(b200):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    b200.lib()      # raises if the library was not built: no CPU fallback
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test the device-side status word must still be 0 (no bounded wait ran out)."""
    yield
    if request.node.get_closest_marker("gpu"):
        import torch
        if torch.cuda.is_available():
            mod = load_package()
            assert mod.device_status() == 0, "a device-side wait timed out"
