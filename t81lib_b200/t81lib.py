"""Drop-in for the hot functions of the reference's pybind11 module ``t81lib``
(python/bindings.cpp:759-1002): same names, argument meaning, return shapes and
exception types, computed on the B200 through ``libt81_b200.so``.

Host inputs (numpy arrays, buffers) are copied to the device, processed there
and copied back, so these calls can replace the reference's one for one; torch
CUDA tensors are used in place with no copies.  There is no CPU implementation.

One additive behaviour: ``gemm_ternary`` also accepts a *dense float* ``B`` of
shape (K, N) instead of packed limbs.  That runs the TRIT-mode contraction
(ternary weights times float activations); packed ``B`` keeps the reference's
LIMB semantics (python/bindings.cpp:769-810, src/linalg/gemm_cpu.cpp:8-71).
"""

from __future__ import annotations

import numpy as np
import torch

from . import _capi, ops

TRITS_PER_LIMB = 48
TRYTES_PER_LIMB = 16
BYTES_PER_LIMB = 16
HAS_CUDA_BACKEND = True
HAS_ROCM_BACKEND = False


def _device() -> torch.device:
    if not _capi.device_available():
        raise RuntimeError(_capi.last_error())
    return torch.device("cuda", torch.cuda.current_device())


def _is_tensor(obj) -> bool:
    return isinstance(obj, torch.Tensor)


def _check_threshold(threshold: float) -> None:
    # python/bindings.cpp:419,463
    if threshold <= 0.0 or threshold > 1.0:
        raise ValueError("threshold must be between 0 (exclusive) and 1")


def _packed_to_device(obj, rows: int, cols: int) -> torch.Tensor:
    """Validate a packed-limb argument like handle_for_packed_object
    (python/bindings.cpp:247-371) and return a CUDA uint8 tensor of rows*cols*16 bytes."""
    if _is_tensor(obj):
        if obj.ndim != 3:
            raise ValueError("packed torch tensors must be 3-dimensional")
        if tuple(obj.shape) != (rows, cols, BYTES_PER_LIMB):
            raise ValueError("packed torch tensor shape must be (rows, cols, bytes_per_limb)")
        if obj.dtype != torch.uint8:
            raise ValueError("packed torch tensors must store uint8 bytes")
        if not obj.is_contiguous():
            raise ValueError("packed torch tensor must be contiguous")
        return obj if obj.is_cuda else obj.to(_device())
    if isinstance(obj, np.ndarray):
        if not obj.flags.c_contiguous:
            raise ValueError("packed limb buffer must use C-style contiguous layout")
        if obj.nbytes != rows * cols * BYTES_PER_LIMB:
            raise ValueError("packed limb buffer byte size mismatch")
        flat = obj.reshape(-1).view(np.uint8) if obj.nbytes else np.zeros(0, np.uint8)
        return torch.from_numpy(flat.copy()).to(_device())
    try:
        view = memoryview(obj)
    except TypeError:
        raise ValueError("packed limbs must come from buffers or torch tensors") from None
    if not view.c_contiguous:
        raise ValueError("packed limb buffer must use C-style contiguous layout")
    if view.nbytes != rows * cols * BYTES_PER_LIMB:
        raise ValueError("packed limb buffer byte size mismatch")
    flat = np.frombuffer(view, dtype=np.uint8) if view.nbytes else np.zeros(0, np.uint8)
    return torch.from_numpy(flat.copy()).to(_device())


def gemm_ternary(A, B, C, M: int, N: int, K: int, alpha: float = 1.0, beta: float = 0.0) -> None:
    """``C = alpha * A @ B + beta * C`` in place on ``C`` (float32, (M, N)); returns None.

    A: packed limbs (M, K/48).  B: packed limbs (K/48, N) for the reference's LIMB
    semantics, or a float array / tensor of shape (K, N) for TRIT semantics."""
    if M < 0 or N < 0 or K < 0:
        raise ValueError("gemm_ternary dimensions must be non-negative")
    if K % TRITS_PER_LIMB != 0:
        raise ValueError("K must be divisible by the limb trit count")
    kl = K // TRITS_PER_LIMB
    dense_b = (_is_tensor(B) and B.is_floating_point()) or (
        isinstance(B, np.ndarray) and B.dtype.kind == "f")
    a_dev = _packed_to_device(A, M, kl)
    if dense_b:
        b_host = B if _is_tensor(B) else torch.from_numpy(np.ascontiguousarray(B))
        if b_host.ndim != 2 or tuple(b_host.shape) != (K, N):
            raise ValueError("dense B must have shape (K, N)")
        b_dev = b_host if b_host.is_cuda else b_host.to(a_dev.device)
    else:
        b_dev = _packed_to_device(B, kl, N)

    # C: torch tensor (used in place when on the device) or a writable float32 buffer
    if _is_tensor(C):
        if C.dtype != torch.float32:
            raise ValueError("buffer must hold float32 elements")
        if C.ndim != 2 or tuple(C.shape) != (M, N):
            raise ValueError("C tensor shape must match (M, N)")
        if not C.is_contiguous():
            raise ValueError("buffer must be C-contiguous")
        c_dev = C if C.is_cuda else C.to(a_dev.device)
        c_host = None if C.is_cuda else C
    else:
        view = memoryview(C)
        if view.itemsize != 4 or view.format not in ("f", "<f", "=f", "@f"):
            raise ValueError("buffer must hold float32 elements")
        if not view.c_contiguous:
            raise ValueError("buffer must be C-contiguous")
        if view.readonly:
            raise ValueError("C buffer must be writable")
        if not ((view.ndim == 2 and tuple(view.shape) == (M, N)) or (view.ndim == 1 and view.shape[0] == M * N)):
            raise ValueError("C tensor shape must match (M, N)")
        c_np = np.frombuffer(view, dtype=np.float32).reshape(M, N)
        c_dev = torch.from_numpy(c_np.copy()).to(a_dev.device)
        c_host = c_np
    if M == 0 or N == 0:
        return None
    if dense_b:
        ops.gemm_trit(a_dev, b_dev, M=M, K=K, layout="kn", C=c_dev, alpha=alpha, beta=beta)
    else:
        ops.gemm_limb(a_dev, b_dev, c_dev, M, N, K, alpha, beta)
    if c_host is not None:
        result = c_dev.cpu()
        if _is_tensor(c_host):
            c_host.copy_(result)
        else:
            c_host[...] = result.numpy()
    return None


def pack_dense_matrix(matrix, threshold: float = 0.5):
    """python/bindings.cpp:460-517.  numpy in -> numpy uint8 (rows, limbs, 16) out;
    a CUDA tensor in -> CUDA tensor out."""
    _check_threshold(threshold)
    if _is_tensor(matrix):
        if matrix.ndim != 2:
            raise ValueError("pack_dense_matrix expects a 2D array")
        on_device = matrix.is_cuda
        src = matrix if on_device else matrix.to(_device())
        if not src.is_floating_point() or src.dtype == torch.float64:
            src = src.to(torch.float32)
        packed, _ = ops.quantize_pack(src, threshold, "fixed")
        return packed if on_device else packed.cpu()
    arr = np.ascontiguousarray(matrix, dtype=np.float32)
    if arr.ndim != 2:
        raise ValueError("pack_dense_matrix expects a 2D array")
    packed, _ = ops.quantize_pack(torch.from_numpy(arr).to(_device()), threshold, "fixed")
    return packed.cpu().numpy()


def quantize_to_trits(values, threshold: float = 0.5):
    """python/bindings.cpp:416-445."""
    _check_threshold(threshold)
    if _is_tensor(values):
        if values.ndim == 0:
            raise ValueError("expected at least one dimension for quantization")
        out = ops.quantize_trits(values if values.is_cuda else values.to(_device()), threshold)
        return out if values.is_cuda else out.cpu()
    arr = np.ascontiguousarray(values, dtype=np.float32)
    if arr.ndim == 0:
        raise ValueError("expected at least one dimension for quantization")
    return ops.quantize_trits(torch.from_numpy(arr).to(_device()), threshold).cpu().numpy()


def dequantize_trits(trits):
    """python/bindings.cpp:447-458: int8 trits -> float32 (a dtype conversion)."""
    if _is_tensor(trits):
        return trits.to(torch.float32)
    return np.ascontiguousarray(trits, dtype=np.int8).astype(np.float32)


def unpack_packed_limbs(packed, rows: int, cols: int):
    """python/bindings.cpp:640-686."""
    if rows < 0 or cols < 0:
        raise ValueError("rows and cols must be non-negative")
    is_t = _is_tensor(packed)
    arr = packed if is_t else torch.from_numpy(np.ascontiguousarray(packed, dtype=np.uint8))
    if arr.ndim != 3:
        raise ValueError("packed limbs must be a 3D array")
    if rows != arr.shape[0]:
        raise ValueError("row count mismatch")
    if arr.shape[2] != BYTES_PER_LIMB:
        raise ValueError("packed limb innermost dimension must equal limb byte width")
    if cols > arr.shape[1] * TRITS_PER_LIMB:
        raise ValueError("cols exceeds packed trit capacity")
    dev = arr if arr.is_cuda else arr.to(_device())
    trits, bad = ops.unpack(dev, rows, cols, count_bad=True)
    if bad:
        # limb::from_bytes (include/t81/core/limb.hpp:160-169) rejects such bytes
        raise ValueError("limb bytes must be valid tryte encodings (0..26)")
    if is_t:
        return trits if packed.is_cuda else trits.cpu()
    return trits.cpu().numpy()
