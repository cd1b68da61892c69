"""Ternary ``nn.Linear`` — counterpart of the reference's ``t81.nn.Linear``
(t81/nn/linear.py:18-125) with the eval forward on the B200 kernels.

Eval mode: the weight is quantised and packed once on the device
(``TernaryTensor.from_float``) and each forward is one fused kernel call —
ternary matmul, optional per-row scale, bias — on the activations where they
live.  Training mode keeps the reference's quantisation-aware forward: a
straight-through ternary quantiser on ``weight / scale`` with a running absmax
scale (t81/nn/linear.py:72-99, t81/qat.py:12-57), in plain PyTorch.
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
    """Forward: the quantised weights.  Backward: identity onto the float weights."""

    @staticmethod
    def forward(ctx, weights: torch.Tensor, quantized: torch.Tensor) -> torch.Tensor:
        return quantized

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        return grad_output, None


def ternary(x: torch.Tensor, threshold: float = 0.45, stochastic: bool = False) -> torch.Tensor:
    """Ternary quantiser with a straight-through gradient (t81/qat.py:50-57): values are
    clamped to [-1, 1]; magnitudes at or above the threshold become their sign, the rest 0.
    With ``stochastic`` a magnitude above the threshold survives with probability
    (|x| - threshold) / (1 - threshold)."""
    threshold = float(max(0.0, min(threshold, 1.0)))
    with torch.no_grad():
        clamped = x.detach().clamp(-1.0, 1.0)
        magnitude = clamped.abs()
        keep = magnitude >= threshold
        if stochastic:
            p = ((magnitude - threshold) / max(1.0 - threshold, 1e-6)).clamp(0.0, 1.0)
            keep = keep & (torch.rand_like(p) < p)
        quantized = torch.where(keep, torch.sign(clamped), torch.zeros_like(clamped))
    return _StraightThrough.apply(x, quantized)


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
        return result

    def configure_qat(self, *, stochastic_rounding: bool) -> None:
        self._stochastic_rounding = stochastic_rounding
