"""The C-ABI library loads without a GPU and exports every symbol include/ashb200.h declares;
compute entry points are not called here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ashb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ashb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = ctypes.CDLL(os.path.join(ROOT, "torch-ash_b200", "libashb200.so"))
    names = _declared()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_argument_errors_without_gpu():
    lib = ctypes.CDLL(os.path.join(ROOT, "torch-ash_b200", "libashb200.so"))
    lib.ashb_last_error_string.restype = ctypes.c_char_p
    out = ctypes.c_void_p()
    # key_dim out of range is rejected before any CUDA call
    rc = lib.ashb_map_create(7, ctypes.c_int64(10), ctypes.c_void_p(16), 0, ctypes.byref(out))
    assert rc == 1 and b"key_dim" in lib.ashb_last_error_string()
    assert lib.ashb_version() >= 1


def test_python_shim_refuses_cpu_tensors():
    import sys

    import pytest
    import torch

    sys.modules.pop("__ash", None)
    saved = list(sys.path)
    try:
        # the real shim, not the oracle stand-in the CPU host-logic tests use
        sys.path.insert(0, os.path.join(ROOT, "torch-ash_b200"))
        import importlib.util

        spec = importlib.util.spec_from_file_location("_real_ash_shim", os.path.join(ROOT, "torch-ash_b200", "__ash.py"))
        shim = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(shim)
        with pytest.raises(RuntimeError, match="CUDA"):
            shim.HashMap(3, 10, torch.arange(10, dtype=torch.int32), torch.device("cpu"))
        e = torch.zeros(2, 8, 1)
        with pytest.raises(RuntimeError, match="CUDA"):
            shim.query_forward(e, torch.zeros(1, 3), torch.zeros(1, dtype=torch.long), torch.zeros(1, dtype=torch.long),
                               torch.ones(1, dtype=torch.bool), torch.zeros(2, 8, dtype=torch.long),
                               torch.zeros(8, 8, dtype=torch.long), torch.zeros(8, 8, dtype=torch.long), 2, "linear")
    finally:
        sys.path[:] = saved
        sys.modules.pop("__ash", None)
