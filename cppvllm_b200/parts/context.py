"""What a step hands to the parts: the flattened batch on the device, and views of cache and state.

A step is a flat list of T tokens from S requests.  Request s owns the tokens cu_seqlens[s] .. cu_seqlens[s+1]
(a portion of a prompt, or one decoded token); its tokens sit at absolute positions positions[t] and, after
the step, its sequence holds kv_lens[s] tokens.  All index tensors are int32 on the device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .base import CacheSpec


@dataclass
class GroupStepView:
    """One cache group's view of the step: where this step's tokens are written and where requests' pages are."""
    block_tables: torch.Tensor      # [S, W] int32; entry = page id, -1 where the request holds no page
    slot_mapping: torch.Tensor      # [T] int32; page id * page_size + offset for each token of the step
    page_size: int
    num_pages: int                  # pages in the pool, not counting the scratch page


@dataclass
class CacheUnitView:
    """One cache unit's pages: pages[page, *spec.page_shape(page_size)]; for attention's keys and values that is
    pages[page, 0 = K | 1 = V, kv_head, slot in page, :]."""
    pages: torch.Tensor
    group: int
    spec: CacheSpec
    writes: bool = True


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    tokens: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    cu_seqlens: torch.Tensor
    kv_lens: torch.Tensor
    state_slots: torch.Tensor
    groups: List[GroupStepView]
    logit_rows: torch.Tensor
    num_logit_rows: int
    # host-side facts about the step (fixed per captured graph)
    q_lens: Optional[List[int]] = None
    max_q_len: int = 1
    max_kv_len: int = 1
    all_decode: bool = False
    extras: dict = field(default_factory=dict)
