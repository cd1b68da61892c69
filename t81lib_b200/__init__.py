"""B200-native packed-ternary matmul path with the t81lib API.

    from t81lib_b200 import t81lib            # pybind-module counterpart
    import t81lib_b200.torch as t81_torch     # TernaryTensor, trit
    from t81lib_b200.nn import Linear         # ternary nn.Linear

All arithmetic runs in ``lib/libt81_b200.so`` (hand-written sm_100a kernels behind
the C ABI of ``include/t81_b200.h``); importing the package fails if that library
has not been built, and every call fails without a B200.
"""

from . import _capi, ops, t81lib  # noqa: F401

__all__ = ["_capi", "ops", "t81lib"]
__version__ = "0.1"
