"""Test configuration: import paths and the ``gpu`` marker.

``-m "not gpu"`` covers the oracle against the golden fixtures, the host logic and
the C ABI's symbols (no compute call without a GPU); ``-m gpu`` are the parity
tests proper and call the CUDA kernels through the C ABI.
"""

from __future__ import annotations

from pathlib import Path
import sys

import pytest

ROOT = Path(__file__).resolve().parent.parent
for path in (ROOT, ROOT / "helion-mlir-xsmm_b200", ROOT / "tests"):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    import torch

    if torch.cuda.is_available():
        # A launch that never returns must fail its own test, not wedge the suite
        # (the kernels' waits are bounded; this is the belt to those braces).
        if config.pluginmanager.hasplugin("timeout"):
            for item in items:
                if "gpu" in item.keywords and item.get_closest_marker("timeout") is None:
                    item.add_marker(pytest.mark.timeout(300))
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def built_library() -> Path:
    """The C-ABI library, built in-tree if it is missing (nvcc cross-compiles without a GPU)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("b200_build", ROOT / "helion-mlir-xsmm_b200" / "csrc" / "build.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    if module.LIB.exists():
        return module.LIB
    return module.build()
