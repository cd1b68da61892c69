"""The C-ABI library builds, loads and exports every function include/*.h declares.
No compute call is made here (no GPU needed)."""

import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(header).read()
        names += re.findall(r"T81B200_API[^;(]*?\b(t81b200_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for required in ("t81b200_quantize_pack", "t81b200_unpack", "t81b200_gemm_limb", "t81b200_gemm_trit",
                     "t81b200_device_available", "t81b200_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol(lib_built):
    lib = ctypes.CDLL(lib_built)
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_python_binding_lists_the_same_symbols(lib_built):
    from t81lib_b200 import _capi
    assert sorted(_capi.EXPORTS) == declared_functions()


def test_no_device_is_reported_not_hidden(lib_built):
    """Without a B200 the calls fail with a message; they never fall back to a CPU path."""
    import torch
    from t81lib_b200 import _capi
    if torch.cuda.is_available():
        assert _capi.device_available()
        return
    assert not _capi.device_available()
    assert "no CPU fallback" in _capi.last_error()
    rc = _capi.lib.t81b200_quantize_pack(None, 0, 4, 4, 4, 0.5, 0, None, None, None)
    assert rc == _capi.ENODEVICE
