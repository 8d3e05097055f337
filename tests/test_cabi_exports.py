"""The built C-ABI library loads without a GPU and exports every symbol include/dflash_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dflash_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dfl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from dflb import pkg
    lib = pkg.lib()
    names = declared_symbols()
    assert len(names) > 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_compute_refuses_loudly_without_a_device():
    from dflb import pkg
    import numpy as np
    if pkg.device_count() > 0:
        return
    try:
        pkg.QMatrix(pkg.Q4_K, 256, 128, np.zeros(128 * 144, dtype=np.uint8))
    except pkg.DflError as e:
        assert e.name == "NO_DEVICE"
    else:
        raise AssertionError("a compute call succeeded without a GPU")
