"""Token embedding (reference model/model_architecture.cpp:78-79,149: a row gather) and the output head
(:81-86,222-226: logits = float32(y W^T), W the embedding table when tied, no bias, no scaling)."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Part, WeightSpec, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    category = "embedding"

    def __init__(self, runtime, prefix="", names=None, *, vocab_size: int, hidden_size: int):
        super().__init__(runtime, prefix, names)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.table = None
        self._gather_table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name("weight"): WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors) -> None:
        self.table = tensors[self.full_name("weight")]
        # a table stored in 32-bit under bf16 activations is gathered from a rounded copy
        self._gather_table = self.table if self.table.dtype == self.rt.dtype else self.table.to(self.rt.dtype)

    def forward(self, tokens, num_tokens: int):
        out = self.rt.workspace.rows("residual", num_tokens, self.hidden_size, self.rt.dtype)
        return ops.embed(out, self._gather_table, tokens[:num_tokens])


@register_part("head", "lm_head")
class LMHead(Part):
    category = "head"

    def __init__(self, runtime, prefix="", names=None, *, vocab_size: int, hidden_size: int):
        super().__init__(runtime, prefix, names)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name("weight"): WeightSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.full_name("weight")]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, y: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """y: [R, D] normed rows; out: float32 [R, V]."""
        return ops.linear(y, self.weight, out=out, out_dtype=torch.float32)
