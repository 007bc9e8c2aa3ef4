"""RMSNorm (reference kernels/fused_ops.cu:61-88): y = T( rnd(x * rsqrt(mean(x^2) + eps)) * w ), the weight
multiplying after the rounding, with no ``1 + w`` offset; and its form fused with the residual add."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Norm, WeightSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, runtime, prefix="", names=None, *, size: int, eps: float, buffer: str = "normed"):
        super().__init__(runtime, prefix, names)
        self.size, self.eps, self.buffer = int(size), float(eps), buffer
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name("weight"): WeightSpec((self.size,), role="vector", init="norm")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.full_name("weight")]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def _out(self, x, out):
        return out if out is not None else self.rt.workspace.rows(self.buffer, x.shape[0], self.size, x.dtype)

    def forward(self, x, out=None):
        return ops.rmsnorm(self._out(x, out), x, self.weight, self.eps)

    def add_forward(self, residual, delta, out=None):
        return ops.add_rmsnorm(self._out(residual, out), residual, delta, self.weight, self.eps)
