import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_package():
    """The package directory is named `esp-dl_b200`, which is not an identifier: import it by path."""
    if "espdl_b200" in sys.modules:
        return sys.modules["espdl_b200"]
    pkg_dir = os.path.join(ROOT, "esp-dl_b200")
    spec = importlib.util.spec_from_file_location(
        "espdl_b200", os.path.join(pkg_dir, "__init__.py"), submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["espdl_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


load_package()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a B200 (run with -m gpu)")
