"""Test configuration.

* ``-m gpu`` tests are the parity tests proper: they drive the CUDA library
  through the C ABI (``__ash`` / ``ash``) on ``cuda:0`` and compare with the CPU
  oracle.
* ``-m "not gpu"`` tests cover the oracle against golden vectors, the host
  logic of the Python layer (running on the oracle stand-in for the native
  module, injected here and only here), and the C-ABI symbol table.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "torch-ash_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

HAS_GPU = torch.cuda.is_available()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # The shared library travels prebuilt to the GPU box; build it only if absent.
    if not os.path.exists(os.path.join(PKG, "libashb200.so")):
        sys.path.insert(0, PKG)
        import build as _build

        _build.build()
    import oracle

    oracle.build()
    if not HAS_GPU:
        # Host-logic tests: the product's Python layer on top of the oracle's
        # stand-in for the native module.  Never done when a GPU is present.
        sys.path.insert(0, os.path.join(ROOT, "oracle", "ref_backend"))


def pytest_collection_modifyitems(config, items):
    if HAS_GPU:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def device():
    return torch.device("cuda:0" if HAS_GPU else "cpu")
