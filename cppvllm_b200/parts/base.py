"""Interfaces of the parts a layer is put together from, and the registry that maps a kind to a class.

Categories: ``mixer`` (token mixing: attention here), ``ffn`` (feed-forward), ``norm``, ``position``
(position encoding), ``block`` (arrangement of mixer, feed-forward and norms with the residual stream),
``embedding`` and ``head``.  A part

* is constructed as ``cls(runtime, prefix=..., names=..., **params)``: all sizes and constants arrive as
  parameters; a part never looks at a model configuration and does not know which model it is in;
* declares its tensors with ``weight_specs()`` (full tensor name -> ``WeightSpec``); the loader checks the
  checkpoint against these and ``bind()`` hands the tensors over; the random-weights writer draws them;
* runs with ``forward`` on the tokens of one step (see each category's class below).

A mixer additionally declares what it keeps between steps: ``cache_spec()`` for keys and values that grow
with the sequence (paged, optionally windowed) and ``state_spec()`` for per-request state of fixed size.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch

# ---- registry ------------------------------------------------------------------------------------------

_REGISTRY: Dict[str, Dict[str, type]] = {c: {} for c in
                                         ("mixer", "ffn", "norm", "position", "block", "embedding", "head")}


def register_part(category: str, kind: str, cls: type = None, replace: bool = False):
    """Register `cls` under (category, kind); usable as a decorator: ``@register_part("mixer", "my_kind")``."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category '{category}'; categories: {sorted(_REGISTRY)}")

    def deco(c):
        if kind in _REGISTRY[category] and not replace:
            raise ValueError(f"{category} kind '{kind}' is already registered")
        _REGISTRY[category][kind] = c
        return c

    return deco(cls) if cls is not None else deco


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        raise ValueError(f"no {category} of kind '{kind}' is registered; registered: "
                         f"{sorted(_REGISTRY.get(category, {}))}") from None


def build_part(category: str, spec, runtime, **extra):
    cls = part_class(category, spec.kind)
    return cls(runtime, prefix=spec.prefix, names=dict(spec.names), **spec.params, **extra)


# ---- declarations ----------------------------------------------------------------------------------------

@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]
    role: str = "matrix"      # "matrix": operand of a matrix product / embedding table (engine dtype, or float32
                              #           if stored so); "vector": norm weights and the like (always float32);
                              # "int_table": integer look-up table (int32)
    init: str = "normal"      # random weights: "normal" = N(0, std), "norm" = 1 + U(-spread, spread)


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token in the paged cache.  A page is one tensor of shape
    `entry_shape[:token_axis] + (page_size,) + entry_shape[token_axis:]` in the engine's element type: the token's entry
    with the page's positions inserted at `token_axis`.  Units with equal specs form one group of pages; the cache
    manager hands out pages and block tables and never looks inside a page.
      attention:   CacheSpec.keys_and_values(kv_heads, head_dim)   pages [2, kv_heads, page, head_dim]
      a latent:    CacheSpec((width,), token_axis=0)                pages [page, width]"""
    entry_shape: Tuple[int, ...]
    token_axis: int = 0
    window: int = 0           # 0 = all positions; w > 0 = only the last w positions are ever read (older pages go back)

    @staticmethod
    def keys_and_values(num_kv_heads: int, head_dim: int, window: int = 0) -> "CacheSpec":
        return CacheSpec((2, int(num_kv_heads), int(head_dim)), token_axis=2, window=int(window))

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        return tuple(self.entry_shape[:self.token_axis]) + (page_size,) + tuple(self.entry_shape[self.token_axis:])

    def elements_per_token(self) -> int:
        n = 1
        for d in self.entry_shape:
            n *= int(d)
        return n


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size: one tensor of this shape and dtype per slot, zeroed at admission."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Workspace:
    """Named activation buffers with fixed addresses, sized once for the largest step (`max_tokens` rows).
    Fixed addresses let decode steps be captured in CUDA graphs; sharing names between layers keeps the
    footprint at one layer's worth."""

    def __init__(self, device, max_tokens: int, max_seqs: int = 0):
        self.device = device
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs or max_tokens
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}

    def rows(self, name: str, n_rows: int, width, dtype: torch.dtype) -> torch.Tensor:
        hit = self._views.get((name, n_rows, width, dtype))       # the same view object for the same request
        if hit is not None:
            return hit
        widths = tuple(width) if isinstance(width, (tuple, list)) else (width,)
        key = f"{name}|{widths}|{dtype}"
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty((self.max_tokens,) + widths, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        if n_rows > self.max_tokens:
            raise ValueError(f"a step of {n_rows} tokens exceeds the workspace of {self.max_tokens}")
        view = buf[:n_rows]
        if not isinstance(width, list):
            if len(self._views) > 4096:
                self._views.clear()
            self._views[(name, n_rows, width, dtype)] = view
        return view

    def other_of_pair(self, name: str, current: torch.Tensor, n_rows: int, width, dtype: torch.dtype) -> torch.Tensor:
        """Two buffers `name` and `name + "_alt"` take turns (a kernel that reads the residual stream in all of its blocks
        while one block writes the new one needs the new one elsewhere): returns the one that `current` does not lie in."""
        first = self.rows(name, n_rows, width, dtype)
        return self.rows(name + "_alt", n_rows, width, dtype) if current.data_ptr() == first.data_ptr() else first

    def flat(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A named scratch buffer of a fixed number of elements (allocated once, at its first use; `zero`: zero-filled)."""
        key = f"{name}|flat|{dtype}"
        buf = self._buffers.get(key)
        if buf is None:
            buf = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        elif buf.numel() < numel:           # never reallocated: captured graphs hold the address
            raise ValueError(f"scratch buffer '{name}' was sized for {buf.numel()} elements, {numel} are asked for")
        return buf


@dataclass
class Runtime:
    """What parts are built against: the device, the activation element type and the shared workspace.
    `plain_kernels`: parts use their plain twin kernels only (the general attention kernel, library products with
    separate norm and activation kernels; no tensor-core attention, no weight-streaming products, no fusions): the
    path to compare the fast kernels with, inside the whole engine."""
    device: torch.device
    dtype: torch.dtype
    workspace: Workspace
    plain_kernels: bool = False


class Part:
    category = ""
    # False for a part whose forward synchronises with the host or allocates per call: a model that holds such a
    # part runs its decode steps eagerly instead of replaying CUDA graphs.
    capturable = True

    def __init__(self, runtime: Runtime, prefix: str = "", names: Optional[Dict[str, str]] = None):
        self.rt = runtime
        self.prefix = prefix
        self.names = names or {}

    def full_name(self, local: str) -> str:
        return self.names.get(local, self.prefix + local)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by weight_specs() (already on the device, in their final dtype)."""

    def weight_bytes(self) -> int:
        """Bytes of weights a decode step reads from this part (for the roofline)."""
        return 0


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, residual: torch.Tensor, delta: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (in place, rounded to the activation type), then the norm of the new residual."""
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"


class Mixer(Part):
    category = "mixer"

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx, cache, state) -> torch.Tensor:
        """x: [T, D] normed activations of this step's tokens.  ctx: StepContext.  cache: a CacheUnitView or
        None.  state: the [num_slots, *shape] tensor of this run entry's per-request state or None (index it
        with ctx.state_slots).  Returns [T, D]."""
        raise NotImplementedError


class FeedForward(Part):
    category = "ffn"

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of a mixer, a feed-forward and their norms around the residual stream."""
    category = "block"

    def forward(self, h, pending, ctx, cache, state):
        """h: residual stream [T, D]; pending: a delta not yet added to h, or None.  Returns (h, pending)."""
        raise NotImplementedError
