"""TEST INFRASTRUCTURE — NOT THE PRODUCT.

numpy front-end to ``liboracle.so`` (the plain-C CPU restatement in
``t81_oracle.c``).  Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU
legs of ``bench.py`` may import this package; the shipped library never does.
Each wrapper names the reference lines its C function follows in
``t81_oracle.h``.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

_i64 = ctypes.c_int64
_f32 = ctypes.c_float
_p = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` (and, where the reference sources are present,
    ``_ref``) through the Makefile beside this file."""
    if force and os.path.exists(_LIB_PATH):
        os.remove(_LIB_PATH)
    subprocess.run(["make", "-C", _HERE, "oracle"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        src = os.path.join(_HERE, "t81_oracle.c")
        if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.t81o_quantize_to_trits.argtypes = [_p, ctypes.c_size_t, _f32, _p]
        L.t81o_pack_trits_rowwise.argtypes = [_p, _i64, _i64, _p]
        L.t81o_pack_trits_columnwise.argtypes = [_p, _i64, _i64, _p]
        L.t81o_pack_dense_matrix.argtypes = [_p, _i64, _i64, _i64, _f32, _p]
        L.t81o_pack_dense_matrix_absmean.argtypes = [_p, _i64, _i64, _i64, _f32, _p, _p]
        L.t81o_unpack_packed_limbs.argtypes = [_p, _i64, _i64, _i64, _p]
        L.t81o_unpack_packed_limbs.restype = ctypes.c_int
        L.t81o_gemm_limb.argtypes = [_p, _p, _p, _i64, _i64, _i64, _f32, _f32]
        L.t81o_gemm_trit.argtypes = [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _f32]
        L.t81o_linear_forward.argtypes = [_p, _p, _p, _p, _p, _i64, _i64, _i64]
        L.t81o_num_threads.restype = ctypes.c_int
        L.t81o_set_num_threads.argtypes = [ctypes.c_int]
        for name in ("t81o_quantize_to_trits", "t81o_pack_trits_rowwise", "t81o_pack_trits_columnwise",
                     "t81o_pack_dense_matrix", "t81o_pack_dense_matrix_absmean", "t81o_gemm_limb",
                     "t81o_gemm_trit", "t81o_linear_forward", "t81o_set_num_threads"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(_p)


def _f32c(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def set_num_threads(n: int) -> None:
    lib().t81o_set_num_threads(int(n))


def num_threads() -> int:
    return lib().t81o_num_threads()


def k_limbs(cols: int) -> int:
    return (cols + 47) // 48


def quantize_to_trits(values, threshold: float = 0.5) -> np.ndarray:
    src = _f32c(values)
    out = np.empty(src.shape, dtype=np.int8)
    lib().t81o_quantize_to_trits(_ptr(src), src.size, threshold, _ptr(out))
    return out


def pack_trits_rowwise(trits) -> np.ndarray:
    t = np.ascontiguousarray(trits, dtype=np.int8)
    rows, cols = t.shape
    out = np.empty((rows, k_limbs(cols), 16), dtype=np.uint8)
    lib().t81o_pack_trits_rowwise(_ptr(t), rows, cols, _ptr(out))
    return out


def pack_trits_columnwise(trits) -> np.ndarray:
    t = np.ascontiguousarray(trits, dtype=np.int8)
    k, cols = t.shape
    out = np.empty((k_limbs(k), cols, 16), dtype=np.uint8)
    lib().t81o_pack_trits_columnwise(_ptr(t), k, cols, _ptr(out))
    return out


def pack_dense_matrix(w, threshold: float = 0.5) -> np.ndarray:
    w = _f32c(w)
    rows, cols = w.shape
    out = np.empty((rows, k_limbs(cols), 16), dtype=np.uint8)
    lib().t81o_pack_dense_matrix(_ptr(w), rows, cols, cols, threshold, _ptr(out))
    return out


def pack_dense_matrix_absmean(w, threshold: float = 0.45):
    w = _f32c(w)
    rows, cols = w.shape
    out = np.empty((rows, k_limbs(cols), 16), dtype=np.uint8)
    scale = np.empty(rows, dtype=np.float32)
    lib().t81o_pack_dense_matrix_absmean(_ptr(w), rows, cols, cols, threshold, _ptr(out), _ptr(scale))
    return out, scale


def unpack_packed_limbs(packed, rows: int, cols: int) -> np.ndarray:
    p = np.ascontiguousarray(packed, dtype=np.uint8)
    kl = p.size // (16 * rows) if rows else 0
    out = np.zeros((rows, cols), dtype=np.int8)
    if lib().t81o_unpack_packed_limbs(_ptr(p), rows, kl, cols, _ptr(out)) != 0:
        raise ValueError("packed limb byte out of range (> 26)")
    return out


def gemm_limb(A, B, C, M: int, N: int, K: int, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    """In-place on a float32 copy of C, which is returned."""
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    C = np.array(C, dtype=np.float32, order="C", copy=True).reshape(M, N)
    lib().t81o_gemm_limb(_ptr(A), _ptr(B), _ptr(C), M, N, K // 48, alpha, beta)
    return C


def gemm_trit(A, B, C, M: int, N: int, K: int, alpha: float = 1.0, beta: float = 0.0,
              b_is_nk: bool = False) -> np.ndarray:
    """A packed (M, ceil(K/48), 16); B dense (K, N) — or (N, K) with
    ``b_is_nk`` — returns (M, N), or (N, M) with ``b_is_nk`` (the Linear layout)."""
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = _f32c(B)
    if b_is_nk:
        C = (np.zeros((N, M), np.float32) if C is None
             else np.array(C, dtype=np.float32, order="C", copy=True).reshape(N, M))
        lib().t81o_gemm_trit(_ptr(A), _ptr(B), _ptr(C), M, N, K, 1, K, 1, M, alpha, beta)
    else:
        C = (np.zeros((M, N), np.float32) if C is None
             else np.array(C, dtype=np.float32, order="C", copy=True).reshape(M, N))
        lib().t81o_gemm_trit(_ptr(A), _ptr(B), _ptr(C), M, N, K, N, 1, N, 1, alpha, beta)
    return C


def linear_forward(W_packed, row_scale, bias, x, in_features: int) -> np.ndarray:
    W = np.ascontiguousarray(W_packed, dtype=np.uint8)
    out_features = W.shape[0]
    x = _f32c(x).reshape(-1, in_features)
    rs = None if row_scale is None else _f32c(row_scale)
    b = None if bias is None else _f32c(bias)
    y = np.empty((x.shape[0], out_features), dtype=np.float32)
    lib().t81o_linear_forward(_ptr(W), _ptr(rs), _ptr(b), _ptr(x), _ptr(y), x.shape[0],
                              out_features, in_features)
    return y


# ---- the four elementwise helpers next to the GEMM in the reference's backend slot ----------------
# src/linalg/gemm_dispatch.cpp:147-222 (cpu_where / cpu_clamp / cpu_lerp / cpu_addcmul): float32
# arrays of equal length, one IEEE float32 operation per source operator (numpy float32 arithmetic
# rounds after every operation, like that code compiled without contraction).


def where(condition, x, y) -> np.ndarray:
    c, x, y = _f32c(condition), _f32c(x), _f32c(y)
    return np.where(c != np.float32(0.0), x, y).astype(np.float32)


def clamp(values, min_value: float, max_value: float) -> np.ndarray:
    v = _f32c(values)
    lo, hi = np.float32(min_value), np.float32(max_value)
    return np.where(v < lo, lo, np.where(v > hi, hi, v)).astype(np.float32)


def lerp(start, end, weight) -> np.ndarray:
    s, e, w = _f32c(start), _f32c(end), _f32c(weight)
    return (s + w * (e - s)).astype(np.float32)


def addcmul(input, tensor1, tensor2, value: float = 1.0) -> np.ndarray:
    a, t1, t2 = _f32c(input), _f32c(tensor1), _f32c(tensor2)
    return (a + (np.float32(value) * t1) * t2).astype(np.float32)


# ---- GGUF ternary block formats (t81/gguf.py:518-662) -------------------------------------------------
# Blocks of 256 weights of one row; a weight is d * (q - 1) with q = trit + 1 and d an fp16 scale.
#   TQ2_0, 66 bytes (_quantize_blocks_tq2, :586-600; _dequantize_blocks_tq2, :653-662)
#   TQ1_0, 54 bytes (_quantize_blocks_tq1, :526-547; _dequantize_blocks_tq1, :603-620)
# Restated for trits that are already known (no float round trip): a block's scale is the row's scale, or 0
# when the block has no non-zero trit (the absmax the reference takes of trit * scale).


def pack_t2(trits) -> np.ndarray:
    """The decode-stream layout of a (rows, cols) trit matrix, as bytes (own format, no reference counterpart;
    the statement in include/t81_b200.h restated): blocks of 32 rows x 192 columns, block (chunk c, row tile T)
    at byte (c * tiles32 + T) * 1536; lane l = 4 g + t owns 12 little-endian 32-bit words at l * 48; word
    6 gr + m // 2 holds registers j = 4 (m % 2) + r: trit h of register r <-> row 32 T + 16 gr + g + 8 (r % 2),
    column 192 c + 48 t + 4 m + 2 (r // 2) + h, its code (01 = +1, 11 = -1, 00 = 0) at bits 15 - 2j, 14 - 2j
    (h = 0) or 31 - 2j, 30 - 2j (h = 1)."""
    trits = np.asarray(trits, dtype=np.int8)
    rows, cols = trits.shape
    tiles32, chunks = (rows + 31) // 32, (cols + 191) // 192
    padded = np.zeros((tiles32 * 32, chunks * 192), np.int8)
    padded[:rows, :cols] = trits
    code = np.where(padded == 1, 1, np.where(padded == -1, 3, 0)).astype(np.uint32)
    out = np.zeros((chunks, tiles32, 32, 12), np.uint32)
    T = np.arange(tiles32)[None, :, None]
    c = np.arange(chunks)[:, None, None]
    lane = np.arange(32)[None, None, :]
    g, t = lane >> 2, lane & 3
    for gr in range(2):
        for m in range(12):
            for r in range(4):
                j = 4 * (m % 2) + r
                row = 32 * T + 16 * gr + g + 8 * (r % 2)
                for h in range(2):
                    col = 192 * c + 48 * t + 4 * m + 2 * (r // 2) + h
                    shift = (30 if h else 14) - 2 * j
                    out[:, :, :, 6 * gr + m // 2] |= code[row, col] << np.uint32(shift)
    return out.astype("<u4").view(np.uint8).reshape(-1)


def tq_encode(trits, row_scale, fmt: str) -> np.ndarray:
    t = np.ascontiguousarray(trits, dtype=np.int8)
    rows, cols = t.shape
    bpr = (cols + 255) // 256
    q = np.ones((rows, bpr * 256), np.uint16)
    q[:, :cols] = t + 1
    q = q.reshape(rows * bpr, 256)
    scale = np.ones(rows, np.float32) if row_scale is None else _f32c(row_scale)
    d = np.repeat(scale, bpr).reshape(rows * bpr, 1)
    d = np.where((q != 1).any(axis=1, keepdims=True), d, np.float32(0.0)).astype(np.float16)
    if fmt == "TQ2_0":
        g = q.reshape(-1, 2, 4, 32)
        qs = (g[:, :, 0] | (g[:, :, 1] << 2) | (g[:, :, 2] << 4) | (g[:, :, 3] << 6)).reshape(-1, 64)
    elif fmt == "TQ1_0":
        w5 = np.array([81, 27, 9, 3, 1], np.uint16).reshape(1, 5, 1)
        qs0 = (q[:, :160].reshape(-1, 5, 32) * w5).sum(axis=1)
        qs1 = (q[:, 160:240].reshape(-1, 5, 16) * w5).sum(axis=1)
        qh = (q[:, 240:].reshape(-1, 4, 4) * w5[:, :4]).sum(axis=1)
        v = np.concatenate([qs0, qs1, qh], axis=1).astype(np.uint32)
        qs = (v * 256 + 242) // 243
    else:
        raise ValueError(fmt)
    out = np.concatenate([qs.astype(np.uint8), d.view(np.uint8).reshape(-1, 2)], axis=1)
    return out.reshape(rows, bpr, -1)


def tq_decode(blocks, rows: int, cols: int, fmt: str):
    """Returns (trits int8 (rows, cols), block scales float32 (rows, blocks per row))."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(rows, -1, 66 if fmt == "TQ2_0" else 54)
    bpr = b.shape[1]
    flat = b.reshape(rows * bpr, -1)
    d = flat[:, -2:].copy().view(np.float16).astype(np.float32).reshape(rows, bpr)
    if fmt == "TQ2_0":
        qs = flat[:, :64].reshape(-1, 2, 1, 32) >> np.array([0, 2, 4, 6], np.uint8).reshape(1, 1, 4, 1)
        q = np.minimum(qs & 3, 2).reshape(-1, 256)
    else:
        p5 = np.array([1, 3, 9, 27, 81], np.uint8).reshape(1, 5, 1)
        a = (flat[:, :32].reshape(-1, 1, 32) * p5).reshape(-1, 160)            # uint8 arithmetic wraps on purpose
        c = (flat[:, 32:48].reshape(-1, 1, 16) * p5).reshape(-1, 80)
        h = (flat[:, 48:52].reshape(-1, 1, 4) * p5[:, :4]).reshape(-1, 16)
        q = (np.concatenate([a, c, h], axis=1).astype(np.uint16) * 3) >> 8
    trits = (q.astype(np.int8) - 1).reshape(rows, bpr * 256)[:, :cols]
    return np.ascontiguousarray(trits), d


# ---- quantisation-aware-training forward (t81/nn/linear.py:72-99, t81/qat.py:12-57) --------------------


def qat_update_scale(weight, existing=None, momentum: float = 0.99) -> np.float32:
    """_update_training_scale: max(max |w|, 1e-6) on the first call, afterwards
    max(existing * momentum + candidate * (1 - momentum), 1e-6), every operation in float32."""
    candidate = np.maximum(np.abs(_f32c(weight)).max(), np.float32(1e-6)).astype(np.float32)
    if existing is None:
        return candidate
    combined = np.float32(existing) * np.float32(momentum) + candidate * np.float32(1.0 - momentum)
    return np.maximum(combined, np.float32(1e-6)).astype(np.float32)


def qat_quantize(weight, scale, threshold: float) -> np.ndarray:
    """_quantize_tensor on weight / scale (deterministic): clamp to [-1, 1], sign where |.| >= threshold."""
    scaled = _f32c(weight) / np.float32(scale)
    clamped = np.clip(scaled, np.float32(-1.0), np.float32(1.0))
    thr = np.float32(max(0.0, min(threshold, 1.0)))
    return np.where(np.abs(clamped) >= thr, np.sign(clamped), 0).astype(np.int8)


def qat_linear(weight, scale, threshold: float, x, bias=None):
    """F.linear(x, quantized * scale, bias) in float64, and the gradients of sum(y * gy) the reference's autograd
    yields: returns a function gy -> (y, grad_x, grad_w, grad_b)."""
    w = _f32c(weight)
    trits = qat_quantize(w, scale, threshold).astype(np.float64)
    w_eff = trits * np.float64(scale)
    xs = np.asarray(x, np.float64)
    y = xs @ w_eff.T + (0.0 if bias is None else np.asarray(bias, np.float64))

    def grads(gy):
        gy = np.asarray(gy, np.float64)
        slope = np.where(np.abs(w / np.float32(scale)) < np.float32(0.5), 2.0, 0.0)  # dorso_round's derivative
        return y, gy @ w_eff, (gy.T @ xs) * slope, gy.sum(axis=0)
    return grads
