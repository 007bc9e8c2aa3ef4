"""A model as data: which parts every layer is made of, with their sizes, and the order in which layers run.

An architecture's builder (for instance models/qwen3.py) turns its typed configuration into a ``ModelSpec``;
the generic ``CausalLM`` (parts/model.py) builds parts from it through the part registry (parts/base.py).
Nothing in a spec is code: kinds are registry keys, parameters are plain numbers, weight locations are
tensor-name prefixes.

* ``PartSpec(kind, params, prefix, names)``: one part.  ``prefix`` is put before the part's local weight
  names (``"model.layers.3.self_attn."`` + ``"q_proj.weight"``); ``names`` overrides single local names with
  full tensor names (a tied output head names the embedding's table).
* ``LayerSpec``: the parts of one layer and the name of their arrangement (``block``).  Layers need not be
  alike: each has its own mixer and feed-forward spec.
* ``RunEntry(layer, cache, writes_cache)``: one item of the run list.  ``layer`` indexes ``layers`` and may
  occur several times (weights shared between runs).  ``cache`` is the id of the cache unit the mixer uses in
  this run; two entries with the same id share keys and values, and the entry with ``writes_cache=False``
  only reads what the other wrote (a layer that reads another layer's cache).  ``None`` means one unit per
  entry, written by it.  Per-request state of fixed size, if the mixer declares any, belongs to the entry.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""
    names: Dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    block: str = "prenorm"
    block_params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class RunEntry:
    layer: int
    cache: Optional[int] = None
    writes_cache: bool = True


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    final_norm: PartSpec
    lm_head: PartSpec
    positions: Dict[str, PartSpec] = field(default_factory=dict)   # shared position encodings by name
    run_order: Optional[List[RunEntry]] = None                      # None: every layer once, in order
    max_positions: int = 0
    eos_token_ids: tuple = ()
    init: Dict[str, float] = field(default_factory=dict)            # defaults for random weights

    def resolved_run_order(self) -> List[RunEntry]:
        order = self.run_order if self.run_order is not None else [RunEntry(i) for i in range(len(self.layers))]
        out = []
        next_free = 1 + max([e.cache for e in order if e.cache is not None], default=-1)
        for e in order:
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"run list names layer {e.layer}, but the model has {len(self.layers)} layers")
            c = e.cache
            if c is None:
                c = next_free
                next_free += 1
            out.append(RunEntry(e.layer, c, e.writes_cache))
        written = set()
        for e in out:
            if e.writes_cache:
                if e.cache in written:
                    raise ValueError(f"cache unit {e.cache} is written by two run entries")
                written.add(e.cache)
            elif e.cache not in written:
                raise ValueError(f"run entry for layer {e.layer} reads cache unit {e.cache} before any entry wrote it")
        return out
