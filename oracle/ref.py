"""TEST INFRASTRUCTURE — NOT THE PRODUCT.

Loader for ``oracle/_ref``: the reference's own pybind11 module ``t81lib``
compiled, unmodified, from the reference sources by ``oracle/Makefile`` (target
``ref``).  Two builds exist: ``avx512f`` (the flag the reference's own
CMakeLists.txt:49-53 adds) and ``generic``; the first is used when the host CPU
reports avx512f, since otherwise it would die on an illegal instruction.
"""

from __future__ import annotations

import importlib.util
import os
import sysconfig

_HERE = os.path.dirname(os.path.abspath(__file__))
_mod = None
_variant = None


def host_has_avx512f() -> bool:
    try:
        with open("/proc/cpuinfo") as fh:
            return "avx512f" in fh.read()
    except OSError:
        return False


def path(variant: str | None = None) -> str:
    variant = variant or ("avx512f" if host_has_avx512f() else "generic")
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    return os.path.join(_HERE, "_ref", variant, "t81lib" + ext)


def available() -> bool:
    return os.path.exists(path())


def variant() -> str:
    return _variant or ("avx512f" if host_has_avx512f() else "generic")


def load():
    """Import and return the reference ``t81lib`` extension module."""
    global _mod, _variant
    if _mod is None:
        _variant = "avx512f" if host_has_avx512f() else "generic"
        p = path(_variant)
        if not os.path.exists(p):
            raise FileNotFoundError(f"{p} missing: run `make -C oracle ref` where the reference is mounted")
        spec = importlib.util.spec_from_file_location("t81lib", p)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    return _mod


def cuda_dir() -> str:
    """Where ``make -C oracle ref_cuda`` puts the reference built with its CUDA backend slot filled
    by this repository's shim (``t81lib`` module and ``ref_cuda_driver``)."""
    return os.path.join(_HERE, "_ref", "cuda")


def load_cuda():
    """Import the reference's ``t81lib`` module built with T81LIB_USE_CUDA=1 against the shim."""
    p = os.path.join(cuda_dir(), "t81lib" + sysconfig.get_config_var("EXT_SUFFIX"))
    if not os.path.exists(p):
        raise FileNotFoundError(f"{p} missing: run `make -C oracle ref_cuda` where the reference is mounted")
    spec = importlib.util.spec_from_file_location("t81lib_cuda_build", p)
    # the extension's init function is PyInit_t81lib whatever name it is loaded under
    spec = importlib.util.spec_from_file_location("t81lib", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
