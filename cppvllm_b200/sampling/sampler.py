"""Sampling of next tokens from float32 logits rows on the device (kernel: csrc/sampling.cu).

Greedy for temperature <= 0, else Gumbel-max at the given temperature, as the reference samples
(kernels/fused_ops.cu:285-378).  The random stream of a row is a function of (row seed, output position, vocab
index) only, so what a request draws does not depend on the batch it is in; the reference keys its generator
by the row's index in the batch and a call counter (fused_ops.cu:330-335; engine/model_runner.cpp:259-260).
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from ..csrc import ops

_MASK = (1 << 64) - 1


def mix_seed(engine_seed: int, request_key: int) -> int:
    """A 64-bit row seed from the engine's seed and a request's key (splitmix64 finaliser)."""
    z = (engine_seed * 0x9E3779B97F4A7C15 + request_key + 0x632BE59BD9B4E019) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


class Sampler:
    """Two sets of buffers (`slot` 0 and 1) so that the samples of one step can still be on their way to the host
    while the next step is being sampled."""

    SLOTS = 2

    def __init__(self, device, max_rows: int):
        self.device = torch.device(device)
        self.max_rows = max_rows
        n = self.SLOTS
        self._host_f = [torch.empty(max_rows, dtype=torch.float32, pin_memory=True) for _ in range(n)]
        self._host_p = [torch.empty(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(n)]
        self._host_s = [torch.empty(max_rows, dtype=torch.int64, pin_memory=True) for _ in range(n)]
        self._temps = [torch.zeros(max_rows, dtype=torch.float32, device=self.device) for _ in range(n)]
        self._pos = [torch.zeros(max_rows, dtype=torch.int32, device=self.device) for _ in range(n)]
        self._seeds = [torch.zeros(max_rows, dtype=torch.int64, device=self.device) for _ in range(n)]
        self._out = [torch.zeros(max_rows, dtype=torch.int32, device=self.device) for _ in range(n)]
        self._out_host = [torch.empty(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(n)]
        self._done = [None] * n
        self._chunks = 32
        self._scratch = torch.empty(max_rows * self._chunks * 2, dtype=torch.float32, device=self.device)
        self.h2d_bytes_last = 0

    def sample(self, logits: torch.Tensor, temps: Sequence[float], seeds: Sequence[int],
               out_positions: Sequence[int]) -> List[int]:
        """logits: [R, V] float32 on the device, one row per entry of the sequences.  Returns R token ids."""
        R = logits.shape[0]
        if R == 0:
            return []
        self.sample_async(logits, temps, seeds, out_positions, slot=0)
        return self.collect(R, slot=0)

    def collect(self, R: int, slot: int = 0) -> List[int]:
        """Wait for the sample_async that last used `slot` and return its R tokens."""
        ev = self._done[slot]
        if ev is not None:
            ev.synchronize()
        else:
            torch.cuda.current_stream().synchronize()
        return self._out_host[slot][:R].tolist()

    def sample_async(self, logits: torch.Tensor, temps: Sequence[float], seeds: Sequence[int],
                     out_positions: Sequence[int], slot: int = 0) -> torch.Tensor:
        """Enqueue the sampling of R rows and the copy of the tokens to pinned host memory; returns the device
        tensor of tokens (int32 [R]) without waiting for it."""
        R = logits.shape[0]
        if R > self.max_rows or len(temps) != R or len(seeds) != R or len(out_positions) != R:
            raise ValueError("sampler: row count does not match its arguments or exceeds its capacity")
        self._host_f[slot].numpy()[:R] = temps
        self._host_p[slot].numpy()[:R] = out_positions
        self._host_s[slot].numpy()[:R] = np.asarray([x if x < (1 << 63) else x - (1 << 64) for x in seeds], dtype=np.int64)
        self._temps[slot][:R].copy_(self._host_f[slot][:R], non_blocking=True)
        self._pos[slot][:R].copy_(self._host_p[slot][:R], non_blocking=True)
        self._seeds[slot][:R].copy_(self._host_s[slot][:R], non_blocking=True)
        # a large vocabulary is searched by several blocks per row: 32 at few rows, fewer at many, so that there are
        # a couple of thousand blocks (one block per row read its 600 KB of logits at about a fifth of the bandwidth)
        chunks = max(1, min(self._chunks, 2048 // max(R, 1))) if logits.shape[1] >= 16384 else 0
        if chunks < 2:
            chunks = 0
        ops.sample(self._out[slot][:R], logits, None, self._temps[slot], self._seeds[slot], self._pos[slot], num_rows=R,
                   scratch=self._scratch if chunks else None, chunks=chunks)
        self._out_host[slot][:R].copy_(self._out[slot][:R], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._done[slot] = ev
        self.h2d_bytes_last = R * (4 + 4 + 8)
        return self._out[slot][:R]
