"""Rotary position encoding tables (reference model/model_architecture.cpp:67-75): inv_freq_i = theta^(-2i/rot),
angle = position * inv_freq in float64, cos and sin stored as float32 [max_positions, rot/2].  The rotation
itself happens inside the mixer's fused projection epilogue, which reads these tables; ``pairing`` says which
elements form a pair: "half" pairs (i, i + rot/2) as the reference does (fused_ops.cu:157-166), "interleaved"
pairs (2i, 2i+1)."""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_part


@register_part("position", "rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, runtime, prefix="", names=None, *, rotary_dim: int, theta: float, max_positions: int,
                 pairing: str = "half"):
        super().__init__(runtime, prefix, names)
        if rotary_dim <= 0 or rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {rotary_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        self.rotary_dim, self.theta, self.max_positions, self.pairing = int(rotary_dim), float(theta), int(max_positions), pairing
        idx = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), idx / self.rotary_dim).reciprocal()
        angle = torch.outer(torch.arange(self.max_positions, dtype=torch.float64), inv_freq)
        self.cos = angle.cos().to(torch.float32).contiguous().to(runtime.device)
        self.sin = angle.sin().to(torch.float32).contiguous().to(runtime.device)

    @property
    def interleaved(self) -> bool:
        return self.pairing == "interleaved"
