"""The C-ABI library loads without a GPU and exports every symbol the header declares (CPU only)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tenmo_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tenmo_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from tenmo_b200 import lib

    assert os.path.exists(lib.LIB_PATH), "libtenmo_cuda.so is not built: run __graft_entry__.build()"
    so = ctypes.CDLL(lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(so, name), f"{name} is declared in include/tenmo_cuda.h but not exported"
    assert sorted(lib.EXPORTS) == names, "tenmo_b200.lib.EXPORTS and the header disagree"


def test_handle_without_gpu_fails_loudly():
    """No CPU fallback: without a usable CUDA device the handle reports why and every op raises."""
    import torch

    from tenmo_b200 import TenmoCuda, TenmoError

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = TenmoCuda(0)
    assert not h.is_initialized() and h.get_error()
    with pytest.raises(TenmoError):
        h.fill(0, 0.0, 1)
    with pytest.raises(TenmoError):
        h.require()


def test_missing_library_is_reported_not_hidden(tmp_path):
    from tenmo_b200 import TenmoCuda, TenmoError

    h = TenmoCuda(0, path=str(tmp_path / "nope.so"))
    assert not h.is_initialized() and "Failed to load" in h.get_error()
    with pytest.raises(TenmoError):
        h.synchronize()
