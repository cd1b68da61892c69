"""Ternary ``nn.Linear`` — counterpart of the reference's ``t81.nn.Linear``
(t81/nn/linear.py:18-125) with the eval forward on the B200 kernels.

Eval mode: the weight is quantised and packed once on the device
(``TernaryTensor.from_float``) and each forward is one fused kernel call —
ternary matmul, optional per-row scale, bias — on the activations where they
live.  Training mode keeps the reference's quantisation-aware forward — the
ternary quantiser with its surrogate gradient on ``weight / scale`` and a running
absmax scale (t81/nn/linear.py:72-99, t81/qat.py:12-57): with the weight on a CUDA
device the scale update, quantise + pack and the product run on the device kernels
(``_FusedQATLinear``); stochastic rounding and CPU weights take the PyTorch form.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch
from torch import nn
from torch.nn import functional as F

from .. import torch as t81_torch

_DEFAULT_THRESHOLD = 0.45


class _StraightThrough(torch.autograd.Function):
    """Forward: the quantised values.  Backward: the gradient goes to the surrogate unchanged."""

    @staticmethod
    def forward(ctx, surrogate: torch.Tensor, quantized: torch.Tensor) -> torch.Tensor:
        return quantized

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        return grad_output, None


def dorso_round(x: torch.Tensor) -> torch.Tensor:
    """The surrogate whose gradient the quantiser passes on (t81/qat.py:28-34): +-1 beyond +-0.5, 2x between,
    so the weight gradient is doubled inside (-0.5, 0.5) and zero outside."""
    one = torch.ones_like(x)
    return torch.where(x >= 0.5, one, torch.where(x <= -0.5, -one, x * 2.0))


def ternary(x: torch.Tensor, threshold: float = 0.45, stochastic: bool = False) -> torch.Tensor:
    """Ternary quantiser with the reference's surrogate gradient (t81/qat.py:12-57): values are clamped to
    [-1, 1]; magnitudes at or above the threshold become their sign, the rest 0.  With ``stochastic`` a
    magnitude above the threshold survives with probability (|x| - threshold) / (1 - threshold)."""
    threshold = float(max(0.0, min(threshold, 1.0)))
    with torch.no_grad():
        clamped = x.detach().clamp(-1.0, 1.0)
        magnitude = clamped.abs()
        keep = magnitude >= threshold
        if stochastic:
            p = ((magnitude - threshold) / max(1.0 - threshold, 1e-6)).clamp(0.0, 1.0)
            keep = keep & (torch.rand_like(p) < p)
        quantized = torch.where(keep, torch.sign(clamped), torch.zeros_like(clamped))
    return _StraightThrough.apply(dorso_round(x), quantized)


class _FusedQATLinear(torch.autograd.Function):
    """Training forward on the device kernels: the weight is quantised with the running scale and packed in one
    pass (``ops.qat_quantize_pack``), the product runs on the packed-trit matmul with the scale as row scale.
    Backward is the reference's (t81/nn/linear.py:72-80 through t81/qat.py:28-57): the input gradient is
    grad @ (trits * scale); the weight gradient is grad^T @ x times the surrogate's slope, 2 where
    |weight / scale| < 0.5 and 0 elsewhere (the scale itself carries no gradient)."""

    @staticmethod
    def forward(ctx, x, weight, bias, scale, threshold):
        from .. import ops
        packed, row_scale = ops.qat_quantize_pack(weight.detach(), threshold, scale)
        rows, cols = weight.shape
        x2 = x.reshape(-1, cols)
        if x2.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            x2 = x2.float()
        y = ops.gemm_trit(packed, x2.detach(), M=rows, K=cols, layout="nk", row_scale=row_scale,
                          bias=None if bias is None else bias.detach())
        ctx.save_for_backward(x2, weight, scale)
        ctx.packed, ctx.has_bias, ctx.x_shape = packed, bias is not None, x.shape
        return y.reshape(*x.shape[:-1], rows)

    @staticmethod
    def backward(ctx, grad_output):
        from .. import ops
        x2, weight, scale = ctx.saved_tensors
        rows, cols = weight.shape
        g = grad_output.reshape(-1, rows)
        grad_x = grad_w = grad_b = None
        if ctx.needs_input_grad[0]:
            w_eff = ops.unpack(ctx.packed, rows, cols).to(g.dtype) * scale.to(g.dtype)
            grad_x = (g @ w_eff).reshape(ctx.x_shape).to(x2.dtype)
        if ctx.needs_input_grad[1]:
            slope = ((weight.detach() / scale).abs() < 0.5).to(weight.dtype) * 2.0
            grad_w = (g.t().to(weight.dtype) @ x2.to(weight.dtype)) * slope
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = g.sum(dim=0)
        return grad_x, grad_w, grad_b, None, None


class Linear(nn.Linear):
    """Balanced-ternary ``nn.Linear``; ``rule`` selects the eval-mode quantiser
    ("fixed": the reference's fixed threshold; "absmean": per-row scaled)."""

    def __init__(
        self,
        in_features: int,
        out_features: int,
        bias: bool = True,
        device: Optional[torch.device] = None,
        dtype: Optional[torch.dtype] = None,
        threshold: float = _DEFAULT_THRESHOLD,
        rule: str = "fixed",
    ) -> None:
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self.ternary_threshold = threshold
        self.ternary_rule = rule
        self.ternary_weight: Optional[t81_torch.TernaryTensor] = None
        self.register_buffer("training_scale", None)
        self._stochastic_rounding = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.training:
            if self.weight.is_cuda and x.is_cuda and not self._stochastic_rounding and self.weight.dtype == torch.float32:
                # fused path: running scale, quantise + pack and the product all on the device kernels
                scale = self._update_training_scale_on_device()
                return _FusedQATLinear.apply(x, self.weight, self.bias, scale, float(max(0.0, min(self.ternary_threshold, 1.0))))
            return F.linear(x, self._quantize_training_weight(), self.bias)
        if self.ternary_weight is None:
            self.ternary_weight = t81_torch.TernaryTensor.from_float(
                self.weight.detach(), threshold=self.ternary_threshold, rule=self.ternary_rule)
        return self._packed_linear(x)

    def _packed_linear(self, x: torch.Tensor) -> torch.Tensor:
        if x.ndim == 3:
            batch, seq, features = x.shape
            return self._packed_linear(x.reshape(batch * seq, features)).reshape(batch, seq, -1)
        if x.ndim != 2:
            raise ValueError("t81.nn.Linear expects 2D or 3D inputs")
        return self.ternary_weight.matmul_input(x, bias=self.bias)

    def _quantize_training_weight(self) -> torch.Tensor:
        scale = self._update_training_scale()
        quantized = ternary(self.weight / scale, threshold=self.ternary_threshold,
                            stochastic=self._stochastic_rounding)
        return quantized * scale

    def _update_training_scale_on_device(self) -> torch.Tensor:
        """``_update_training_scale`` as one reduction kernel: no host synchronisation, the scale stays on the
        device.  ``training_scale`` keeps its meaning (a 0-dim float32 tensor holding the running scale)."""
        from .. import ops
        device = self.weight.device
        state = self.__dict__.get("_qat_state")
        if state is None or state.device != device:
            state = torch.zeros(4, dtype=torch.float32, device=device)
            existing = self.training_scale
            if existing is not None:  # carried over from the PyTorch path or another device
                state[0] = existing.to(device=device, dtype=torch.float32)
                state[3] = 1.0
            self.__dict__["_qat_state"] = state
        scale = ops.qat_update_scale(self.weight.detach(), state)
        self.training_scale = state[0]
        return scale

    def _update_training_scale(self) -> torch.Tensor:
        device = self.weight.device
        candidate = self.weight.detach().abs().amax().clamp(min=1e-6).to(device=device, dtype=torch.float32)
        existing = self.training_scale
        if existing is None or existing.device != device:
            self.training_scale = candidate.detach()
            return self.training_scale
        momentum = 0.99
        combined = existing.to(dtype=torch.float32) * momentum + candidate * (1.0 - momentum)
        self.training_scale = combined.clamp(min=1e-6).detach()
        return self.training_scale

    def extra_repr(self) -> str:
        base = super().extra_repr()
        if self.ternary_threshold != _DEFAULT_THRESHOLD:
            return f"{base}, threshold={self.ternary_threshold}"
        return base

    def train(self, mode: bool = True) -> "Linear":
        if mode and getattr(self, "_t81_float_released", False):
            raise RuntimeError("this layer's float weight was released at conversion; it can only run in eval mode")
        if mode:
            self.ternary_weight = None
        return super().train(mode)

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        normalized = OrderedDict()
        for key, value in state_dict.items():
            if key in {"weight", "bias"} and value.is_floating_point() and value.dtype in {torch.bfloat16, torch.float16}:
                value = value.to(torch.float32)
            normalized[key] = value
        result = super().load_state_dict(normalized, strict=strict, assign=assign)
        self.ternary_weight = None
        self.training_scale = None
        self.__dict__.pop("_qat_state", None)
        return result

    def configure_qat(self, *, stochastic_rounding: bool) -> None:
        self._stochastic_rounding = stochastic_rounding
