"""ctypes binding of ``libt81_b200.so`` (declared in ``include/t81_b200.h``).

The library is the only compute path: if it is missing or cannot be loaded the
import of this module fails, and if no B200 is present every call raises.
"""

from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libt81_b200.so")

OK, EINVAL, ENODEVICE, ECUDA, EWORKSPACE, EALIGN, ELIMIT = 0, -1, -2, -3, -4, -5, -6
F32, BF16, F16 = 0, 1, 2
RULE_FIXED, RULE_ABSMEAN = 0, 1
LAYOUT_KN, LAYOUT_NK = 0, 1
STATIC_SCRATCH_BYTES = 16 << 20

MAX_PEERS = 7       # T81B200_MAX_PEERS
SYNC_WORDS = 256    # T81B200_SYNC_WORDS

EXPORTS = (
    "t81b200_device_available", "t81b200_last_error", "t81b200_version", "t81b200_quantize_pack",
    "t81b200_quantize_trits", "t81b200_unpack", "t81b200_gemm_limb", "t81b200_gemm_limb_host",
    "t81b200_gemm_trit", "t81b200_gemm_trit_host", "t81b200_gemm_trit_static", "t81b200_gemm_trit_workspace_bytes", "t81b200_kernel_status",
    "t81b200_copy_columns", "t81b200_gemm_trit_peers", "t81b200_exchange_wait", "t81b200_hint_independent",
    "t81b200_gemm_limb_auto", "t81b200_gemm_trit_auto", "t81b200_elementwise", "t81b200_elementwise_auto",
    "t81b200_release_staging", "t81b200_exchange_signal", "t81b200_gemm_trit_grouped", "t81b200_t2_bytes", "t81b200_pack_t2", "t81b200_prefers_streaming", "t81b200_gemm_trit_t2", "t81b200_gemm_trit_t2_peers", "t81b200_tq_bytes", "t81b200_packed_to_tq", "t81b200_tq_to_packed",
    "t81b200_qat_update_scale", "t81b200_qat_quantize_pack",
)
TQ1_0, TQ2_0 = 0, 1
T2_MAX_TOKENS = 128  # T81B200_T2_MAX_ROWS
MAX_GROUP = 3       # T81B200_MAX_GROUP
EW_WHERE, EW_CLAMP, EW_LERP, EW_ADDCMUL = 0, 1, 2, 3


class T81B200Error(RuntimeError):
    """A CUDA-side failure reported by the library (ECUDA, ENODEVICE, ...)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"t81_b200 error {code}: {message}")
        self.code = code


def _load() -> ctypes.CDLL:
    from . import build as _build
    if _build._stale():
        # sources changed since the library was built (or it was never built): rebuild in-tree
        try:
            _build.build()
        except Exception as exc:  # no nvcc, compile error: there is nothing to fall back to
            raise ImportError(
                f"{LIB_PATH} is missing or out of date and could not be built: {exc} "
                "(there is no fallback implementation)") from exc
    lib = ctypes.CDLL(LIB_PATH)
    i64, f32, vp, ci = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int
    lib.t81b200_device_available.restype = ci
    lib.t81b200_last_error.restype = ctypes.c_char_p
    lib.t81b200_version.restype = ctypes.c_char_p
    lib.t81b200_quantize_pack.argtypes = [vp, ci, i64, i64, i64, f32, ci, vp, vp, vp]
    lib.t81b200_quantize_trits.argtypes = [vp, i64, f32, vp, vp]
    lib.t81b200_unpack.argtypes = [vp, i64, i64, i64, vp, vp, vp]
    lib.t81b200_gemm_limb.argtypes = [vp, vp, vp, i64, i64, i64, f32, f32, vp]
    lib.t81b200_gemm_limb_host.argtypes = [vp, vp, vp, i64, i64, i64, f32, f32]
    lib.t81b200_gemm_trit.argtypes = [vp, vp, vp, ci, ci, i64, vp, vp, ci, i64, i64, i64, i64, f32, f32,
                                      vp, ctypes.c_size_t, vp]
    lib.t81b200_gemm_trit_static.argtypes = [vp, vp, vp, ci, ci, i64, vp, vp, ci, i64, i64, i64, i64, f32, f32, vp]
    lib.t81b200_gemm_trit_host.argtypes = [vp, vp, vp, i64, i64, i64, f32, f32]
    lib.t81b200_gemm_trit_workspace_bytes.argtypes = [ci, ci, ci, i64, i64, i64]
    lib.t81b200_gemm_trit_workspace_bytes.restype = ctypes.c_size_t
    lib.t81b200_kernel_status.argtypes = [ci]
    lib.t81b200_copy_columns.argtypes = [vp, i64, vp, i64, i64, i64, vp]
    lib.t81b200_gemm_trit_peers.argtypes = [vp, vp, vp, ci, ci, i64, vp, vp, ci, i64, i64, i64, i64, f32, f32,
                                            vp, ctypes.c_size_t, ci, ctypes.POINTER(vp), vp, ctypes.POINTER(vp), vp]
    lib.t81b200_exchange_wait.argtypes = [vp, ci, vp]
    lib.t81b200_hint_independent.argtypes = [ci]
    lib.t81b200_gemm_limb_auto.argtypes = [vp, vp, vp, i64, i64, i64, f32, f32]
    lib.t81b200_gemm_trit_auto.argtypes = [vp, vp, vp, i64, i64, i64, f32, f32]
    lib.t81b200_elementwise.argtypes = [ci, vp, vp, vp, vp, i64, f32, f32, vp]
    lib.t81b200_elementwise_auto.argtypes = [ci, vp, vp, vp, vp, i64, f32, f32]
    lib.t81b200_qat_update_scale.argtypes = [vp, ci, i64, i64, i64, f32, vp, vp]
    lib.t81b200_qat_quantize_pack.argtypes = [vp, ci, i64, i64, i64, f32, vp, vp, vp, vp]
    lib.t81b200_tq_bytes.argtypes = [ci, i64, i64]
    lib.t81b200_tq_bytes.restype = i64
    lib.t81b200_packed_to_tq.argtypes = [vp, vp, i64, i64, ci, vp, vp]
    lib.t81b200_tq_to_packed.argtypes = [vp, i64, i64, ci, vp, vp, vp]
    lib.t81b200_gemm_trit_grouped.argtypes = [ci, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp),
                                              ctypes.POINTER(vp), ctypes.POINTER(i64), vp, ci, i64, ci, i64, i64, i64,
                                              f32, f32, vp]
    lib.t81b200_exchange_signal.argtypes = [vp, ctypes.POINTER(vp), ci, vp]
    lib.t81b200_prefers_streaming.argtypes = [i64, i64, i64]
    lib.t81b200_gemm_trit_t2.argtypes = lib.t81b200_gemm_trit_grouped.argtypes
    lib.t81b200_gemm_trit_t2_peers.argtypes = [vp, vp, vp, vp, i64, vp, ci, i64, ci, i64, i64, i64, f32, f32, ci,
                                               ctypes.POINTER(vp), vp, ctypes.POINTER(vp), vp]
    lib.t81b200_t2_bytes.argtypes = [i64, i64]
    lib.t81b200_t2_bytes.restype = i64
    lib.t81b200_pack_t2.argtypes = [vp, i64, i64, vp, vp]
    lib.t81b200_hint_independent.restype = None
    for name in EXPORTS:
        fn = getattr(lib, name)
        if fn.restype is ctypes.c_int and name not in ("t81b200_device_available",):
            fn.restype = ci
    return lib


lib = _load()


def last_error() -> str:
    return lib.t81b200_last_error().decode()


class LimitError(ValueError):
    """A size beyond a stated fixed maximum of the entry point that was called (ELIMIT)."""


def check(code: int) -> None:
    """Map a return code to the exception the reference raises for that failure:
    argument problems are ``ValueError`` (pybind's value_error / std::invalid_argument),
    runtime failures are ``RuntimeError``."""
    if code == OK:
        return
    msg = last_error()
    if code == ELIMIT:
        raise LimitError(msg)
    if code in (EINVAL, EALIGN, EWORKSPACE):
        raise ValueError(msg)
    raise T81B200Error(code, msg)


def device_available() -> bool:
    return bool(lib.t81b200_device_available())


def kernel_status(reset: bool = False) -> int:
    """Status word of the tensor-core kernel (0 = fine); synchronises the device."""
    return lib.t81b200_kernel_status(1 if reset else 0)


def version() -> str:
    return lib.t81b200_version().decode()
