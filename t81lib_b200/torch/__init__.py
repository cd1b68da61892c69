"""B200 counterpart of the reference's ``t81.torch`` (t81/torch/__init__.py):
``TernaryTensor``, ``trit`` / ``TritDtype`` and the ``nn.Module.to(dtype=trit)`` /
``nn.Linear.forward`` patches, with the packed weights, the quantiser and the
matmul all resident on the GPU.

Differences from the reference, all on purpose:
  * tensors stay on the device (the reference moves everything to the CPU and
    warns); CPU inputs are moved to the current CUDA device;
  * ``matmul_input`` multiplies the ternary weights with the *float* activations
    (TRIT mode).  The reference thresholds the activations to trits too and
    multiplies whole limbs as integers (t81/torch/__init__.py:257-276), which
    overflows fp32 at real sizes;
  * ``matmul_input`` takes the ``bias=`` keyword that t81/nn/linear.py:62 already
    passes, and fuses it (and the optional per-row scale) into the kernel;
  * ``from_float(..., rule="absmean")`` offers a per-row-scaled quantiser next to
    the reference's fixed-threshold rule (the default).
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional, Sequence

import torch
from torch import nn

from .. import _capi, ops


class TritDtype:
    __slots__ = ()

    def __new__(cls) -> "TritDtype":
        return super().__new__(cls)

    def __repr__(self) -> str:
        return "t81.trit"


trit = TritDtype()


def _clamp_threshold(threshold: float) -> float:
    # t81/torch/__init__.py:45
    return float(max(0.0, min(threshold, 0.9999)))


def _to_device_float(tensor: torch.Tensor) -> torch.Tensor:
    """Counterpart of _to_cpu_float (t81/torch/__init__.py:53-65) with the direction
    reversed: the data ends up on a CUDA device in a float dtype the kernels read."""
    if tensor.is_meta:
        raise NotImplementedError(
            "t81.trit does not support meta tensors; load weights on CPU or disable offload."
        )
    tensor = tensor.detach()
    if not tensor.is_cuda:
        if not _capi.device_available():
            raise RuntimeError(_capi.last_error())
        tensor = tensor.to(torch.device("cuda", torch.cuda.current_device()))
    if tensor.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        tensor = tensor.to(torch.float32)
    return tensor


# Decode-sized products (1..16 activation rows) of a TernaryTensor run on a second copy of the weight in the
# decode-stream layout (ops.pack_t2), made on first use: 0.25 byte per weight on top of the 0.33 of the limbs.
# False keeps every product on the limb layout.
DECODE_STREAM_LAYOUT = True


class TernaryTensor(torch.Tensor):
    """A (rows, cols) ternary matrix stored as packed limbs on the GPU.

    ``_packed`` is a CUDA uint8 tensor (rows, k_limbs, 16) in the reference's limb
    layout, byte for byte what ``t81lib.pack_dense_matrix`` produces.  The tensor
    body itself carries no data (a one-element buffer expanded to the logical
    shape), so a TernaryTensor costs 2.67 bits per weight, not 32."""

    __slots__ = (
        "_packed",
        "_row_scale",
        "_rows",
        "_k_actual",
        "_k_limbs",
        "_float_source",
        "_base_device",
        "_threshold",
        "_rule",
        "_t2",
    )

    def __new__(
        cls,
        packed: torch.Tensor,
        shape: tuple[int, int],
        *,
        k_actual: int,
        k_limbs: int,
        float_source: Optional[torch.Tensor] = None,
        threshold: float = 0.5,
        row_scale: Optional[torch.Tensor] = None,
        rule: str = "fixed",
    ) -> "TernaryTensor":
        body = torch.empty(1, dtype=torch.float32, device=packed.device).expand(shape)
        tensor = torch.Tensor._make_subclass(cls, body, False)
        tensor._packed = packed
        tensor._row_scale = row_scale
        tensor._rows = shape[0]
        tensor._k_actual = k_actual
        tensor._k_limbs = k_limbs
        tensor._float_source = float_source
        tensor._base_device = packed.device
        tensor._threshold = _clamp_threshold(threshold)
        tensor._rule = rule
        tensor._t2 = None  # the decode-stream layout, made by the first decode-sized product; False: does not apply
        return tensor

    @property
    def dtype(self) -> TritDtype:  # type: ignore[override]
        return trit

    @property
    def packed(self) -> torch.Tensor:
        return self._packed

    @property
    def row_scale(self) -> Optional[torch.Tensor]:
        return self._row_scale

    def __repr__(self) -> str:  # noqa: D105
        return f"TernaryTensor(shape={tuple(self.shape)}, trits_per_row={self._k_actual})"

    @staticmethod
    def _ensure_int2d(tensor: torch.Tensor) -> torch.Tensor:
        if tensor.ndim != 2:
            raise ValueError("t81.trit tensors currently only support 2D matrices")
        return tensor

    @classmethod
    def from_float(cls, source: torch.Tensor, quantize: bool = True, threshold: float = 0.5,
                   rule: str = "fixed") -> "TernaryTensor":
        """t81/torch/__init__.py:214-231, on the device.  ``quantize=False`` takes
        ``source`` as already holding -1/0/+1 values."""
        tensor = cls._ensure_int2d(source)
        dev_float = _to_device_float(tensor)
        rows, cols = dev_float.shape
        k_limbs = (cols + 47) // 48
        if quantize:
            packed, scale = ops.quantize_pack(dev_float, _clamp_threshold(threshold), rule)
        else:
            # values are trits already: any threshold in (0, 1] reproduces them
            packed, scale = ops.quantize_pack(dev_float.to(torch.float32), 0.5, "fixed")
        return cls(packed, (rows, cols), k_actual=cols, k_limbs=k_limbs, float_source=dev_float,
                   threshold=threshold, row_scale=scale, rule=rule if quantize else "fixed")

    def update_from_float(self, source: torch.Tensor) -> None:
        """t81/torch/__init__.py:233-239: re-quantise into the existing packed buffer."""
        dev_float = _to_device_float(self._ensure_int2d(source))
        if tuple(dev_float.shape) != (self._rows, self._k_actual):
            raise ValueError("source shape does not match the ternary tensor")
        ops.quantize_pack(dev_float, self._threshold, self._rule, out=self._packed,
                          row_scale_out=self._row_scale)
        self._float_source = dev_float
        self._t2 = None

    def to_trits(self) -> torch.Tensor:
        """int8 (rows, cols) trits (the inverse of the packer)."""
        return ops.unpack(self._packed, self._rows, self._k_actual)

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        w = self.to_trits().to(dtype)
        if self._row_scale is not None:
            w = w * self._row_scale.to(dtype)[:, None]
        return w

    def _streams(self, tokens: int) -> bool:
        """17..128 activation rows: slices of the streaming kernel or tensor-core tiles (the library's estimate)."""
        return 16 < tokens <= _capi.T2_MAX_TOKENS and bool(_capi.lib.t81b200_prefers_streaming(self._rows, tokens, self._k_actual))

    def matmul_input(self, input: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``input @ W.T (+ bias)`` for activations (tokens, cols) -> (tokens, rows).
        t81/torch/__init__.py:241-246 with the bias keyword of t81/nn/linear.py:62."""
        if input.ndim != 2:
            raise ValueError("t81.trit linear helpers expect 2D activations")
        needs_grad = torch.is_grad_enabled() and (input.requires_grad or (bias is not None and bias.requires_grad))
        if not needs_grad and input.is_cuda and input.device == self._base_device:
            # inference fast path: no autograd node, no device shuffling — one kernel call
            if input.shape[1] != self._k_actual:
                raise ValueError("rhs dimension does not match ternary weight width")
            if DECODE_STREAM_LAYOUT and (1 <= input.shape[0] <= 16 or self._streams(input.shape[0])) and self._t2 is not False and self._rows > 0 and self._k_actual > 0:
                # decode-sized: the weight in the decode-stream layout (made once, a quarter fewer bytes to stream)
                if self._t2 is None:
                    self._t2 = ops.pack_t2(self._packed, self._rows, self._k_actual)
                try:
                    x = input if input.stride(1) == 1 else input.contiguous()
                    if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                        raise ValueError(f"x must be float32, bfloat16 or float16, got {x.dtype}")
                    if bias is not None and (bias.dtype != torch.float32 or bias.device != x.device or not bias.is_contiguous()):
                        bias = bias.detach().to(device=x.device, dtype=torch.float32).contiguous()
                    return ops.gemm_trit_t2_one(self._t2, self._rows, x, self._k_actual, self._row_scale, bias, out_dtype)
                except _capi.LimitError:
                    self._t2 = False  # a contraction too long for that kernel: the limb layout serves it
            return ops.gemm_trit(self._packed, input, M=self._rows, K=self._k_actual, layout="nk",
                                 row_scale=self._row_scale, bias=bias, out_dtype=out_dtype)
        return _TernaryLinearFunction.apply(self, input, bias, out_dtype)

    @classmethod
    def __torch_function__(cls, func: Callable, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in {torch.matmul, torch.mm}:
            lhs, rhs = args
            if isinstance(lhs, TernaryTensor):
                return _TernaryGemmFunction.apply(lhs, rhs)
        # metadata reads (shape, device, size(), ...) act on the data-less body; anything
        # that would compute with it is refused, as in the reference
        if getattr(func, "__name__", "") == "__get__" or func in _METADATA_FUNCS:
            with torch._C.DisableTorchFunctionSubclass():
                return func(*args, **kwargs)
        return NotImplemented

    def _compute_gemm(self, rhs: torch.Tensor) -> torch.Tensor:
        """(rows, cols) @ rhs (cols, N) -> (rows, N); t81/torch/__init__.py:264-276."""
        if rhs.ndim != 2:
            raise ValueError("t81.trit linear helpers expect 2D activations")
        if rhs.shape[0] != self._k_actual:
            raise ValueError("rhs dimension does not match ternary weight width")
        return ops.gemm_trit(self._packed, rhs, M=self._rows, K=self._k_actual, layout="kn",
                             row_scale=self._row_scale)


_METADATA_FUNCS = {torch.Tensor.size, torch.Tensor.dim, torch.Tensor.numel, torch.Tensor.stride,
                   torch.Tensor.is_floating_point, torch.Tensor.is_contiguous}


def _as_device_activations(x: torch.Tensor, device: torch.device) -> torch.Tensor:
    x = _to_device_float(x)
    return x if x.device == device else x.to(device)


class _TernaryGemmFunction(torch.autograd.Function):
    """torch.matmul(TernaryTensor, rhs): t81/torch/__init__.py:279-304."""

    @staticmethod
    def forward(ctx, ternary_weight: TernaryTensor, rhs: torch.Tensor) -> torch.Tensor:
        ctx.ternary = ternary_weight
        ctx.rhs_device = rhs.device
        ctx.rhs_dtype = rhs.dtype
        dev_rhs = _as_device_activations(rhs, ternary_weight._base_device)
        output = ternary_weight._compute_gemm(dev_rhs)
        if rhs.device != output.device:
            output = output.to(rhs.device)
        return output

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        # grad_rhs = T(W)^T @ grad_out, the dense form the reference uses (:292-304)
        w = ctx.ternary.dequantize(torch.float32)
        grad = w.transpose(-2, -1).matmul(grad_output.to(device=w.device, dtype=torch.float32))
        return None, grad.to(device=ctx.rhs_device, dtype=ctx.rhs_dtype)


class _TernaryLinearFunction(torch.autograd.Function):
    """matmul_input: activations (tokens, K) in their natural layout, fused scale + bias."""

    @staticmethod
    def forward(ctx, ternary_weight: TernaryTensor, x: torch.Tensor, bias, out_dtype):
        ctx.ternary = ternary_weight
        ctx.x_device = x.device
        ctx.x_dtype = x.dtype
        ctx.has_bias = bias is not None
        if x.shape[1] != ternary_weight._k_actual:
            raise ValueError("rhs dimension does not match ternary weight width")
        dev_x = _as_device_activations(x, ternary_weight._base_device)
        output = ops.gemm_trit(ternary_weight._packed, dev_x, M=ternary_weight._rows,
                               K=ternary_weight._k_actual, layout="nk",
                               row_scale=ternary_weight._row_scale, bias=bias, out_dtype=out_dtype)
        if x.device != output.device:
            output = output.to(x.device)
        return output

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        w = ctx.ternary.dequantize(torch.float32)
        g = grad_output.to(device=w.device, dtype=torch.float32)
        grad_x = g.matmul(w).to(device=ctx.x_device, dtype=ctx.x_dtype)
        grad_bias = g.sum(dim=0) if ctx.has_bias else None
        return None, grad_x, grad_bias, None


# ---- nn.Module.to(dtype=trit) and nn.Linear.forward patches (t81/torch/__init__.py:115-164,307-335)


def _extract_dtype_arg(args: Sequence[Any], kwargs: Mapping[str, Any]):
    dtype = kwargs.get("dtype")
    if dtype is not None:
        return dtype
    for arg in args:
        if isinstance(arg, (torch.dtype, TritDtype)):
            return arg
    return None


def _sync_ternary_weights(module: nn.Module, _: Sequence[Any]) -> None:
    """Keep the packed cache consistent with the float weights before a forward.
    The reference re-quantises on every call; here a parameter's version counter and
    storage pointer tell whether it changed since the last pack."""
    cache: Dict[str, TernaryTensor] = getattr(module, "_t81_ternary_cache", {})
    stamps: Dict[str, tuple] = module.__dict__.setdefault("_t81_ternary_stamps", {})
    for name, ternary in cache.items():
        source = getattr(module, name)
        stamp = (source._version, source.data_ptr(), source.device)
        if stamps.get(name) != stamp:
            ternary.update_from_float(source)
            stamps[name] = stamp


def _apply_ternary_conversion(module: nn.Module) -> None:
    for submodule in module.modules():
        if hasattr(submodule, "_t81_ternary_cache"):
            continue
        cache: Dict[str, TernaryTensor] = {}
        stamps: Dict[str, tuple] = {}
        for name, parameter in submodule.named_parameters(recurse=False):
            if parameter.ndim != 2:
                continue
            threshold = getattr(submodule, "ternary_threshold", getattr(submodule, "threshold", 0.5))
            cache[name] = TernaryTensor.from_float(parameter.detach(), threshold=threshold)
            stamps[name] = (parameter._version, parameter.data_ptr(), parameter.device)
        if cache:
            setattr(submodule, "_t81_ternary_cache", cache)
            submodule.__dict__["_t81_ternary_stamps"] = stamps
            if not hasattr(submodule, "_t81_hook_handle"):
                handle = submodule.register_forward_pre_hook(_sync_ternary_weights)
                setattr(submodule, "_t81_hook_handle", handle)


_original_module_to = nn.Module.to
_original_linear_forward = nn.Linear.forward


def _ternary_module_to(self, *args, **kwargs):
    dtype = _extract_dtype_arg(args, kwargs)
    if dtype is trit:
        args = tuple(a for a in args if a is not trit)
        kwargs = {k: v for k, v in kwargs.items() if v is not trit}
        module = _original_module_to(self, *args, **kwargs) if (args or kwargs) else self
        _apply_ternary_conversion(module)
        return module
    return _original_module_to(self, *args, **kwargs)


def _ternary_linear_forward(self, input: torch.Tensor) -> torch.Tensor:
    cache: Dict[str, TernaryTensor] = getattr(self, "_t81_ternary_cache", {})
    ternary = cache.get("weight")
    if ternary is not None:
        _sync_ternary_weights(self, ())
        lead = input.shape[:-1]
        output = ternary.matmul_input(input.reshape(-1, input.shape[-1]), bias=self.bias)
        return output.reshape(*lead, -1)
    return _original_linear_forward(self, input)


def install_patches() -> None:
    """Apply the two global patches the reference applies at import time."""
    nn.Module.to = _ternary_module_to
    nn.Linear.forward = _ternary_linear_forward


def remove_patches() -> None:
    nn.Module.to = _original_module_to
    nn.Linear.forward = _original_linear_forward


install_patches()

__all__ = ["trit", "TernaryTensor", "TritDtype", "install_patches", "remove_patches"]
