"""The C-ABI library loads and exports every symbol the public header declares (no GPU needed)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "deltanet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dn_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from deltanet_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "build the library first (deltanet-tpu_b200/csrc/build.sh)"
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
    # every symbol the Python binding uses is declared in the header
    assert set(_lib.EXPORTED) <= set(names)


def test_status_strings_and_shape_checks():
    from deltanet_b200 import _lib
    lib = _lib.lib()
    assert lib.dn_version() >= 1
    assert lib.dn_status_string(0) == b"ok"
    s = _lib.Shape(B=1, L=256, Hk=2, Hv=4, K=64, V=64, chunk=64, g_heads=2, g_cols=64, b_heads=2, b_cols=64,
                   w_heads=4, w_cols=64, qkv_dtype=0, gate_dtype=0, precision=0, flags=0, scale=0.125)
    e = _lib.Exec()
    assert lib.dn_exec_view(s, e) == 0
    assert (e.H, e.Vw, e.G, e.NC) == (2, 128, 2, 4)
    assert lib.dn_residual_bytes(s) > 0 and lib.dn_scratch_bytes(s, 1, 1) > lib.dn_scratch_bytes(s, 1, 0)
    s.K = 96
    assert lib.dn_exec_view(s, e) == 1          # DN_ERR_BAD_SHAPE
    s.K, s.g_heads = 64, 4                      # a gate per value head switches to Hv exec heads
    assert lib.dn_exec_view(s, e) == 0 and (e.H, e.Vw, e.G) == (4, 64, 1)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest
    from deltanet_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or eager fallback"):
        _lib.lib()
