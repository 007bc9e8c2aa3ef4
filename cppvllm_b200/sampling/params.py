"""Per-request sampling options.  ``temperature``, ``max_tokens`` and ``ignore_eos`` are the reference's
``SamplingParams`` with its defaults (engine/sequence.h:18-24): temperature 1.0 (<= 0 means greedy), 256 new
tokens, stop at an end-of-sequence token.  ``seed`` is added: a request with a seed draws the same tokens in
every run and in every batch; without one, the engine's seed and the request's number are used."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 256
    ignore_eos: bool = False
    seed: Optional[int] = None

    def __post_init__(self):
        if self.max_tokens < 0:
            raise ValueError("max_tokens must be >= 0")
