"""The generic causal language model: an embedding, a run list of blocks, a final norm and an output head,
all built from a ``ModelSpec`` through the part registry.  It holds no architecture-specific code; an
architecture contributes only its spec (see models/qwen3.py).

``forward(ctx, caches, states)`` runs exactly the tokens of the step, reading and writing the cache units it is
given, and returns float32 logits for the rows listed in ``ctx.logit_rows`` (any tokens of the step, not only
last ones; the reference computes one row per sequence whether it samples or not, model_architecture.cpp:232-235).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import CacheSpec, Runtime, StateSpec, WeightSpec, build_part, part_class
from .spec import ModelSpec, RunEntry


class CausalLM:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.hidden_size, self.vocab_size = spec.hidden_size, spec.vocab_size
        self.positions = {name: build_part("position", ps, runtime) for name, ps in spec.positions.items()}
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = []
        for ls in spec.layers:
            mixer_extra = {}
            mparams = dict(ls.mixer.params)
            pos_name = mparams.pop("position", None)
            mixer_cls = part_class("mixer", ls.mixer.kind)
            if pos_name is not None:
                if pos_name not in self.positions:
                    raise ValueError(f"mixer names position encoding '{pos_name}', which the spec does not define")
                mixer_extra["position"] = self.positions[pos_name]
            mixer = mixer_cls(runtime, prefix=ls.mixer.prefix, names=dict(ls.mixer.names), **mparams, **mixer_extra)
            ffn = build_part("ffn", ls.ffn, runtime)
            mixer_norm = build_part("norm", ls.mixer_norm, runtime)
            ffn_norm = build_part("norm", ls.ffn_norm, runtime)
            block_cls = part_class("block", ls.block)
            self.blocks.append(block_cls(runtime, mixer=mixer, ffn=ffn, mixer_norm=mixer_norm, ffn_norm=ffn_norm,
                                         **ls.block_params))
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.lm_head, runtime)
        self.run_order: List[RunEntry] = spec.resolved_run_order()
        self._check_shared_caches()

    @property
    def capturable(self) -> bool:
        return all(p.capturable for p in self.all_parts())

    # ---- what the model keeps between steps ------------------------------------------------------------
    def cache_units(self) -> Dict[int, CacheSpec]:
        """cache unit id -> spec, taken from the mixer of the entry that writes the unit."""
        units = {}
        for e in self.run_order:
            cs = self.blocks[e.layer].mixer.cache_spec()
            if cs is not None and e.writes_cache:
                units[e.cache] = cs
        return units

    def state_specs(self) -> List[Optional[StateSpec]]:
        """One entry per item of the run list: the fixed-size per-request state its mixer wants, or None."""
        return [self.blocks[e.layer].mixer.state_spec() for e in self.run_order]

    def _check_shared_caches(self) -> None:
        units = self.cache_units()
        for e in self.run_order:
            cs = self.blocks[e.layer].mixer.cache_spec()
            if cs is None or e.writes_cache:
                continue
            w = units.get(e.cache)
            if w is None or (w.entry_shape, w.token_axis) != (cs.entry_shape, cs.token_axis):
                raise ValueError(f"layer {e.layer} reads cache unit {e.cache}, whose entries have another shape")

    # ---- weights -------------------------------------------------------------------------------------
    def all_parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head
        yield from self.positions.values()

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for p in self.all_parts():
            for name, ws in p.weight_specs().items():
                if name in specs and specs[name].shape != ws.shape:
                    raise ValueError(f"tensor '{name}' is declared with shapes {specs[name].shape} and {ws.shape}")
                specs.setdefault(name, ws)
        return specs

    def ignorable_weights(self):
        """Tensors a checkpoint may hold although the model does not read them: the head's own table when
        the head is tied to the embedding."""
        own = self.spec.lm_head.prefix + "weight"
        return [own] if self.head.full_name("weight") != own else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.all_parts():
            p.bind(tensors)

    def decode_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every run entry's layer once (a layer run twice is read
        twice), the final norm and the head; the embedding table only as the head when tied."""
        total = 0
        for e in self.run_order:
            total += sum(p.weight_bytes() for p in self.blocks[e.layer].parts())
        return total + self.final_norm.weight_bytes() + self.head.weight_bytes()

    # ---- step ----------------------------------------------------------------------------------------
    def forward_hidden(self, ctx, caches, states):
        h = self.embedding.forward(ctx.tokens, ctx.num_tokens)
        pending = None
        for i, e in enumerate(self.run_order):
            h, pending = self.blocks[e.layer].forward(h, pending, ctx, caches.get(i), states.get(i))
        return h, pending

    def forward(self, ctx, caches, states, logits_out: torch.Tensor) -> torch.Tensor:
        h, pending = self.forward_hidden(ctx, caches, states)
        R = ctx.num_logit_rows
        ws = self.rt.workspace
        rows_h = ops.gather_rows(ws.rows("head_rows", R, self.hidden_size, h.dtype), h, ctx.logit_rows)
        normed = ws.rows("head_normed", R, self.hidden_size, h.dtype)
        if pending is not None:
            rows_p = ops.gather_rows(ws.rows("head_pending", R, self.hidden_size, h.dtype), pending, ctx.logit_rows)
            self.final_norm.add_forward(rows_h, rows_p, out=normed)
        else:
            self.final_norm.forward(rows_h, out=normed)
        return self.head.forward(normed, logits_out[:R])
