import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def load_pkg():
    """Imports the package directory `llama-vulkan_b200` (not a valid module
    name because of the hyphen) under the name llama_vulkan_b200."""
    name = "llama_vulkan_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "llama-vulkan_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def pkg():
    return load_pkg()


@pytest.fixture(scope="session")
def oracle():
    import oracle_bind
    return oracle_bind.load()


@pytest.fixture(scope="session")
def gpu(pkg):
    """One lv_ctx on cuda:0 for the whole GPU test session."""
    ctx = pkg.Context(0)
    yield ctx
    ctx.close()
