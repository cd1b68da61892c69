"""Tensor-level entry points over the C ABI.

Every function takes CUDA tensors, queues work on torch's current stream and
returns CUDA tensors.  torch is used for device memory and streams only; all
arithmetic happens in ``libt81_b200.so``.
"""

from __future__ import annotations

import contextlib
import ctypes
from typing import Optional, Tuple

import torch

from . import _capi

TRITS_PER_LIMB = 48
BYTES_PER_LIMB = 16

_DTYPES = {torch.float32: _capi.F32, torch.bfloat16: _capi.BF16, torch.float16: _capi.F16}
_RULES = {"fixed": _capi.RULE_FIXED, "absmean": _capi.RULE_ABSMEAN}


def k_limbs(cols: int) -> int:
    return (cols + TRITS_PER_LIMB - 1) // TRITS_PER_LIMB


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")


def _dtype_code(t: torch.Tensor, name: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"{name} must be float32, bfloat16 or float16, got {t.dtype}") from None


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Per-device scratch buffer, grown on demand and reused by later calls on the
    same stream order."""
    if nbytes == 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


@contextlib.contextmanager
def independent_of_previous():
    """While active, every ``gemm_trit`` call issued by this thread promises that it reads nothing the
    previous kernel on its stream wrote and writes nothing that kernel touches (k and v behind q, up
    behind gate: same input, different outputs).  Decode-sized calls then start while their
    predecessor still runs; completion order is unchanged, so later calls need no extra care.
    A hinted kernel lets its own successor start at once, so in a run of consecutive hinted calls
    each must be independent of every kernel back to and including the last unhinted one."""
    _capi.lib.t81b200_hint_independent(1)
    try:
        yield
    finally:
        _capi.lib.t81b200_hint_independent(0)


def quantize_pack(w: torch.Tensor, threshold: float = 0.5, rule: str = "fixed",
                  out: Optional[torch.Tensor] = None,
                  row_scale_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Threshold-quantise a 2-D weight and pack it row-wise into limbs.

    Returns ``(packed uint8 (rows, k_limbs, 16), row_scale float32 (rows,) or None)``.
    """
    if w.ndim != 2:
        raise ValueError("pack_dense_matrix expects a 2D array")
    _require_cuda(w, "w")
    if rule not in _RULES:
        raise ValueError(f"unknown quantiser rule {rule!r}")
    if w.stride(1) != 1 and w.numel() > 0:
        w = w.contiguous()
    rows, cols = w.shape
    kl = k_limbs(cols)
    with torch.cuda.device(w.device):
        packed = out if out is not None else torch.empty((rows, kl, 16), dtype=torch.uint8, device=w.device)
        if out is not None and (out.numel() != rows * kl * 16 or out.dtype != torch.uint8 or not out.is_contiguous()):
            raise ValueError("packed output buffer has the wrong size")
        scale = None
        if rule == "absmean":
            scale = row_scale_out if row_scale_out is not None else torch.empty(rows, dtype=torch.float32, device=w.device)
        ld = w.stride(0) if rows > 1 else max(cols, 1)
        _capi.check(_capi.lib.t81b200_quantize_pack(
            _ptr(w), _dtype_code(w, "w"), rows, cols, max(ld, cols), float(threshold), _RULES[rule],
            _ptr(packed), _ptr(scale), _stream(w.device)))
    return packed, scale


def quantize_trits(values: torch.Tensor, threshold: float = 0.5) -> torch.Tensor:
    _require_cuda(values, "values")
    src = values.to(torch.float32).contiguous()
    out = torch.empty(src.shape, dtype=torch.int8, device=src.device)
    with torch.cuda.device(src.device):
        _capi.check(_capi.lib.t81b200_quantize_trits(_ptr(src), src.numel(), float(threshold), _ptr(out),
                                                     _stream(src.device)))
    return out


def unpack(packed: torch.Tensor, rows: int, cols: int, count_bad: bool = False):
    """Packed limbs -> int8 trits (rows, cols).  With ``count_bad`` also returns the
    number of bytes above 26 that were met."""
    _require_cuda(packed, "packed")
    packed = packed.contiguous()
    kl = packed.numel() // (16 * rows) if rows else 0
    trits = torch.empty((rows, cols), dtype=torch.int8, device=packed.device)
    bad = torch.zeros(1, dtype=torch.int32, device=packed.device) if count_bad else None
    with torch.cuda.device(packed.device):
        _capi.check(_capi.lib.t81b200_unpack(_ptr(packed), rows, kl, cols, _ptr(trits), _ptr(bad),
                                             _stream(packed.device)))
    if count_bad:
        return trits, int(bad.item())
    return trits


def gemm_limb(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, M: int, N: int, K: int,
              alpha: float = 1.0, beta: float = 0.0) -> None:
    """LIMB mode, in place on C (float32 (M, N) CUDA)."""
    for t, name in ((A, "A"), (B, "B"), (C, "C")):
        _require_cuda(t, name)
    with torch.cuda.device(C.device):
        _capi.check(_capi.lib.t81b200_gemm_limb(_ptr(A), _ptr(B), _ptr(C), M, N, K // TRITS_PER_LIMB,
                                                float(alpha), float(beta), _stream(C.device)))


def gemm_trit(packed: torch.Tensor, B: torch.Tensor, *, M: int, K: int, layout: str,
              row_scale: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
              C: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
              out_dtype: Optional[torch.dtype] = None, peers=None, sync=None) -> torch.Tensor:
    """TRIT mode.  ``layout="kn"``: B is (K, N), result (M, N).  ``layout="nk"``:
    B is (N, K) (one token per row), result (N, M).

    ``peers``: tensors with C's shape, strides and dtype whose memory lives on other GPUs of
    the node (mapped into this process); every element of C is written to them too.  ``sync``:
    an object with ``local_ptr`` and ``slot_ptrs`` (see ``nn.sharded.ExchangeFlags``): the call then
    waits on the device for the peers' previous stores and signals its own."""
    _require_cuda(packed, "packed")
    _require_cuda(B, "B")
    if B.ndim != 2:
        raise ValueError("gemm_trit expects a 2D dense operand")
    if B.stride(1) != 1 and B.numel() > 0:
        B = B.contiguous()
    if layout == "kn":
        if B.shape[0] != K:
            raise ValueError("rhs dimension does not match ternary weight width")
        N = B.shape[1]
        c_shape, code = (M, N), _capi.LAYOUT_KN
    elif layout == "nk":
        if B.shape[1] != K:
            raise ValueError("rhs dimension does not match ternary weight width")
        N = B.shape[0]
        c_shape, code = (N, M), _capi.LAYOUT_NK
    else:
        raise ValueError(f"unknown layout {layout!r}")
    if C is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs C")
        C = torch.empty(c_shape, dtype=out_dtype or B.dtype, device=B.device)
    else:
        _require_cuda(C, "C")
        if tuple(C.shape) != c_shape or C.stride(1) != 1:
            raise ValueError(f"C must have shape {c_shape} with unit inner stride")
    b_code, c_code = _dtype_code(B, "B"), _dtype_code(C, "C")
    ldb = B.stride(0) if B.shape[0] > 1 else max(B.shape[1], 1)
    ldc = C.stride(0) if C.shape[0] > 1 else max(C.shape[1], 1)
    dev = B.device
    rs = row_scale
    if rs is not None and (rs.dtype != torch.float32 or rs.device != dev or not rs.is_contiguous()):
        rs = rs.to(device=dev, dtype=torch.float32).contiguous()
    bs = bias
    if bs is not None and (bs.dtype != torch.float32 or bs.device != dev or not bs.is_contiguous()):
        bs = bs.detach().to(device=dev, dtype=torch.float32).contiguous()
    direct = b_code == _capi.BF16 and code == _capi.LAYOUT_NK  # no scratch needed
    if peers:
        for t in peers:
            if tuple(t.shape) != tuple(C.shape) or t.stride() != C.stride() or t.dtype != C.dtype:
                raise ValueError("peer results must have C's shape, strides and dtype")
        ptrs = (ctypes.c_void_p * len(peers))(*[t.data_ptr() for t in peers])
        with torch.cuda.device(dev):
            need = 0 if direct else _capi.lib.t81b200_gemm_trit_workspace_bytes(b_code, code, c_code, M, N, K)
            ws = _workspace(dev, need)
            _capi.check(_capi.lib.t81b200_gemm_trit_peers(
                _ptr(packed), _ptr(rs), _ptr(B), b_code, code, ldb, _ptr(bs), _ptr(C), c_code, ldc,
                M, N, K, float(alpha), float(beta), _ptr(ws), 0 if ws is None else ws.numel(), len(peers), ptrs,
                None if sync is None else sync.local_ptr, None if sync is None else sync.slot_ptrs, _stream(dev)))
        return C
    if direct and dev.index == torch.cuda.current_device():
        _capi.check(_capi.lib.t81b200_gemm_trit(
            packed.data_ptr(), _ptr(rs), B.data_ptr(), b_code, code, ldb, _ptr(bs), C.data_ptr(), c_code, ldc,
            M, N, K, float(alpha), float(beta), None, 0, torch.cuda.current_stream(dev).cuda_stream))
        return C
    with torch.cuda.device(dev):
        need = 0 if direct else _capi.lib.t81b200_gemm_trit_workspace_bytes(b_code, code, c_code, M, N, K)
        ws = _workspace(dev, need)
        _capi.check(_capi.lib.t81b200_gemm_trit(
            _ptr(packed), _ptr(rs), _ptr(B), b_code, code, ldb, _ptr(bs), _ptr(C), c_code, ldc,
            M, N, K, float(alpha), float(beta), _ptr(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return C


def pack_t2(packed: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Packed limbs -> the decode-stream layout (two bits per trit in tensor-core fragment order), uint8 of
    ``t2_bytes(rows, cols)`` bytes on the same device.  Made once per weight; ``gemm_trit_t2`` multiplies it."""
    _require_cuda(packed, "packed")
    packed = packed.contiguous()
    if packed.dtype != torch.uint8 or packed.numel() != rows * ((cols + 47) // 48) * 16:
        raise ValueError("packed does not hold rows x ceil(cols/48) limbs")
    out = torch.empty(int(_capi.lib.t81b200_t2_bytes(rows, cols)), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _capi.check(_capi.lib.t81b200_pack_t2(_ptr(packed), rows, cols, _ptr(out), _stream(packed.device)))
    return out


def gemm_trit_t2_one(t2: torch.Tensor, M: int, x: torch.Tensor, K: int, row_scale: Optional[torch.Tensor] = None,
                     bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``gemm_trit_t2`` for one matrix with as little host work as the call allows (the kernel runs a few
    microseconds: list handling and conversions would outweigh it).  ``x`` is (1..16 tokens, K) with unit column
    stride on ``t2``'s device; ``row_scale`` and ``bias`` are contiguous float32 on that device or None."""
    tokens = x.shape[0]
    dev = x.device
    C = torch.empty((tokens, M), dtype=out_dtype or x.dtype, device=dev)
    vp = ctypes.c_void_p
    a = vp(t2.data_ptr())
    c = vp(C.data_ptr())
    m = ctypes.c_int64(M)
    rs = None if row_scale is None else ctypes.byref(vp(row_scale.data_ptr()))
    bs = None if bias is None else ctypes.byref(vp(bias.data_ptr()))
    args = (1, ctypes.byref(a), rs, bs, ctypes.byref(c), ctypes.byref(m), x.data_ptr(), _DTYPES[x.dtype],
            x.stride(0) if tokens > 1 else max(K, 1), _DTYPES[C.dtype], M, tokens, K, 1.0, 0.0,
            torch.cuda.current_stream(dev).cuda_stream)
    if torch.cuda.current_device() == dev.index:
        rc = _capi.lib.t81b200_gemm_trit_t2(*args)
    else:
        with torch.cuda.device(dev):
            rc = _capi.lib.t81b200_gemm_trit_t2(*args)
    if rc:
        _capi.check(rc)
    return C


def gemm_trit_t2(t2, rows, x: torch.Tensor, *, K: int, row_scales=None, biases=None, outs=None,
                 out_dtype: Optional[torch.dtype] = None, alpha: float = 1.0, beta: float = 0.0, peers=None, sync=None):
    """``gemm_trit_grouped`` on matrices in the decode-stream layout: ``t2`` is a list of ``pack_t2`` results,
    ``rows`` their row counts, ``x`` (1..128 tokens, K).  One kernel launch per 16 tokens.  ``peers`` / ``sync`` (one matrix
    only, ``outs`` given): as in ``gemm_trit`` — the result is also stored into the peers' tensors."""
    if peers:
        if len(t2) != 1 or outs is None:
            raise ValueError("peer stores take one matrix and an explicit result tensor")
        _require_cuda(x, "x")
        if x.ndim != 2 or x.shape[1] != K or not 1 <= x.shape[0] <= 16:
            raise ValueError("the decode-stream layout serves 1 to 16 tokens of width K")
        if x.stride(1) != 1:
            x = x.contiguous()
        C, dev, tokens, M = outs[0], x.device, x.shape[0], int(rows[0])
        if tuple(C.shape) != (tokens, M) or C.stride(1) != 1:
            raise ValueError("the result must be (tokens, rows) with unit column stride")
        for t in peers:
            if tuple(t.shape) != tuple(C.shape) or t.stride() != C.stride() or t.dtype != C.dtype:
                raise ValueError("peer results must have the local result's shape, strides and dtype")
        f32 = lambda t: None if t is None else t.detach().to(device=dev, dtype=torch.float32).contiguous()  # noqa: E731
        scale = f32(row_scales[0]) if row_scales else None
        bias = f32(biases[0]) if biases else None
        ptrs = (ctypes.c_void_p * len(peers))(*[t.data_ptr() for t in peers])
        ldb = x.stride(0) if tokens > 1 else max(K, 1)
        ldc = C.stride(0) if tokens > 1 else max(M, 1)
        with torch.cuda.device(dev):
            _capi.check(_capi.lib.t81b200_gemm_trit_t2_peers(
                _ptr(t2[0]), _ptr(scale), _ptr(bias), _ptr(C), M, _ptr(x), _dtype_code(x, "x"), ldb, _dtype_code(C, "out"), ldc,
                tokens, K, float(alpha), float(beta), len(peers), ptrs, None if sync is None else sync.local_ptr,
                None if sync is None else sync.slot_ptrs, _stream(dev)))
        return outs
    return gemm_trit_grouped(t2, x, K=K, row_scales=row_scales, biases=biases, outs=outs, out_dtype=out_dtype,
                             alpha=alpha, beta=beta, _t2_rows=[int(r) for r in rows])


def gemm_trit_grouped(packed, x: torch.Tensor, *, K: int, row_scales=None, biases=None, outs=None,
                      out_dtype: Optional[torch.dtype] = None, alpha: float = 1.0, beta: float = 0.0, _t2_rows=None):
    """TRIT mode for up to ``_capi.MAX_GROUP`` weight matrices that share their activations (q/k/v, gate/up):
    ``x`` is (tokens, K); returns the list of (tokens, rows_i) results.  With at most 16 tokens the whole
    group is one kernel launch.  ``outs`` may give the result tensors (same dtype, same leading stride)."""
    n = len(packed)
    if not 1 <= n <= _capi.MAX_GROUP:
        raise ValueError(f"between 1 and {_capi.MAX_GROUP} matrices per group")
    _require_cuda(x, "x")
    if x.ndim != 2 or x.shape[1] != K:
        raise ValueError("rhs dimension does not match ternary weight width")
    if x.stride(1) != 1 and x.numel() > 0:
        x = x.contiguous()
    dev, tokens = x.device, x.shape[0]
    rows = _t2_rows if _t2_rows is not None else [int(p.shape[0]) for p in packed]
    for p in packed:
        _require_cuda(p, "packed")
    if _t2_rows is not None and not 1 <= tokens <= _capi.T2_MAX_TOKENS:
        raise ValueError(f"the decode-stream layout serves 1 to {_capi.T2_MAX_TOKENS} tokens")
    if outs is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs outs")
        # one allocation, so that every result has the same leading stride
        whole = torch.empty((tokens, sum(rows)), dtype=out_dtype or x.dtype, device=dev)
        outs, lo = [], 0
        for r in rows:
            outs.append(whole[:, lo:lo + r])
            lo += r
    ldcs = {(o.stride(0) if o.shape[0] > 1 else None) for o in outs} - {None}
    if len(ldcs) > 1 or any(o.stride(1) != 1 or tuple(o.shape) != (tokens, r) or o.dtype != outs[0].dtype
                            for o, r in zip(outs, rows)):
        raise ValueError("grouped results must be (tokens, rows_i) tensors of one dtype with one leading stride")
    ldc = ldcs.pop() if ldcs else max(rows)
    vp = ctypes.c_void_p

    def f32(t):
        if t is None:
            return None
        if t.dtype != torch.float32 or t.device != dev or not t.is_contiguous():
            t = t.detach().to(device=dev, dtype=torch.float32).contiguous()
        return t
    scales = [f32(t) for t in (row_scales or [None] * n)]
    bs = [f32(t) for t in (biases or [None] * n)]
    arr = lambda ts: (vp * n)(*[None if t is None else t.data_ptr() for t in ts])  # noqa: E731
    ldb = x.stride(0) if tokens > 1 else max(K, 1)
    with torch.cuda.device(dev):
        entry = _capi.lib.t81b200_gemm_trit_grouped if _t2_rows is None else _capi.lib.t81b200_gemm_trit_t2
        _capi.check(entry(
            n, arr(packed), arr(scales), arr(bs), arr(outs), (ctypes.c_int64 * n)(*rows), _ptr(x), _dtype_code(x, "x"),
            ldb, _dtype_code(outs[0], "out"), ldc, tokens, K, float(alpha), float(beta), _stream(dev)))
    return outs


_TQ = {"TQ1_0": _capi.TQ1_0, "TQ2_0": _capi.TQ2_0}


def packed_to_tq(packed: torch.Tensor, rows: int, cols: int, fmt: str = "TQ2_0",
                 row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed limbs (+ per-row scale) -> GGUF TQ1_0 / TQ2_0 block payload, uint8 (rows, ceil(cols/256), 54 | 66),
    on the device; the trits are carried over exactly (t81/gguf.py:518-600 without the float round trip)."""
    _require_cuda(packed, "packed")
    if fmt not in _TQ:
        raise ValueError(f"unknown block format {fmt!r}")
    packed = packed.contiguous()
    nbytes = _capi.lib.t81b200_tq_bytes(_TQ[fmt], rows, cols)
    per_block = 66 if fmt == "TQ2_0" else 54
    out = torch.empty((rows, (cols + 255) // 256, per_block), dtype=torch.uint8, device=packed.device)
    assert out.numel() == nbytes
    rs = row_scale
    if rs is not None and (rs.dtype != torch.float32 or rs.device != packed.device or not rs.is_contiguous()):
        rs = rs.to(device=packed.device, dtype=torch.float32).contiguous()
    with torch.cuda.device(packed.device):
        _capi.check(_capi.lib.t81b200_packed_to_tq(_ptr(packed), _ptr(rs), rows, cols, _TQ[fmt], _ptr(out), _stream(packed.device)))
    return out


def tq_to_packed(blocks: torch.Tensor, rows: int, cols: int, fmt: str = "TQ2_0"):
    """GGUF TQ1_0 / TQ2_0 block payload -> (packed limbs uint8 (rows, ceil(cols/48), 16), block scales fp32
    (rows, ceil(cols/256))), on the device."""
    _require_cuda(blocks, "blocks")
    if fmt not in _TQ:
        raise ValueError(f"unknown block format {fmt!r}")
    blocks = blocks.contiguous()
    if blocks.numel() != _capi.lib.t81b200_tq_bytes(_TQ[fmt], rows, cols):
        raise ValueError("block payload size does not match (rows, cols)")
    packed = torch.empty((rows, k_limbs(cols), 16), dtype=torch.uint8, device=blocks.device)
    scales = torch.empty((rows, (cols + 255) // 256), dtype=torch.float32, device=blocks.device)
    with torch.cuda.device(blocks.device):
        _capi.check(_capi.lib.t81b200_tq_to_packed(_ptr(blocks), rows, cols, _TQ[fmt], _ptr(packed), _ptr(scales),
                                                   _stream(blocks.device)))
    return packed, scales


def qat_update_scale(weight: torch.Tensor, state: torch.Tensor, momentum: float = 0.99) -> torch.Tensor:
    """Running absmax scale of a QAT layer on the device (t81/nn/linear.py:82-99).  ``state`` is the layer's
    4-float CUDA buffer (zeros before the first call); returns the one-element view that holds the scale."""
    _require_cuda(weight, "weight")
    if weight.ndim != 2 or weight.stride(1) != 1:
        raise ValueError("qat_update_scale expects a 2D weight with unit inner stride")
    if state.dtype != torch.float32 or state.numel() != 4 or state.device != weight.device:
        raise ValueError("state must be 4 float32 values on the weight's device")
    rows, cols = weight.shape
    with torch.cuda.device(weight.device):
        _capi.check(_capi.lib.t81b200_qat_update_scale(_ptr(weight), _dtype_code(weight, "weight"), rows, cols,
                                                       weight.stride(0) if rows > 1 else max(cols, 1), float(momentum),
                                                       _ptr(state), _stream(weight.device)))
    return state[:1]


def qat_quantize_pack(weight: torch.Tensor, threshold: float, scale: torch.Tensor):
    """Quantise ``weight / scale`` with the training rule (t81/qat.py:12-25, deterministic) and pack it; ``scale`` is a
    one-element CUDA tensor.  Returns (packed limbs, row_scale filled with the scale)."""
    _require_cuda(weight, "weight")
    if weight.ndim != 2 or weight.stride(1) != 1:
        raise ValueError("qat_quantize_pack expects a 2D weight with unit inner stride")
    rows, cols = weight.shape
    packed = torch.empty((rows, k_limbs(cols), 16), dtype=torch.uint8, device=weight.device)
    row_scale = torch.empty(rows, dtype=torch.float32, device=weight.device)
    with torch.cuda.device(weight.device):
        _capi.check(_capi.lib.t81b200_qat_quantize_pack(_ptr(weight), _dtype_code(weight, "weight"), rows, cols,
                                                        weight.stride(0) if rows > 1 else max(cols, 1), float(threshold),
                                                        _ptr(scale), _ptr(packed), _ptr(row_scale), _stream(weight.device)))
    return packed, row_scale
