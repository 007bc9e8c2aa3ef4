"""Grouped-query attention over the paged cache, with optional per-head RMSNorm of q and k and optional
rotary position encoding (reference model/model_architecture.cpp:155-178):

    qkv = x Wqkv^T                      Wqkv = rows(q_proj) over rows(k_proj) over rows(v_proj), no bias
    q, k <- rotate(headnorm(q)), rotate(headnorm(k));  k, v written to this step's slots of the cache pages
    att_t = softmax_j(scale * q_t . k_j) v_j  over the request's positions lo..p_t   (causal; lo = 0 or window edge)
    y = att Wo^T

Prompt portions and decoded tokens run through the same code: every token attends to its request's pages,
which already hold the step's own keys.  A step of decoded tokens only takes a shorter way through the same
arithmetic: one kernel norms, rotates, writes the cache and attends (`fuse_decode_attention`).  All sizes are parameters; `scale` defaults to 1/sqrt(head_dim)
(model_architecture.cpp:134).  The part does not know how many layers exist or which model it serves.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import CacheSpec, Mixer, WeightSpec, register_part


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qk_norm: bool = True, qk_norm_eps: float = 1e-6, window: int = 0,
                 scale: Optional[float] = None, position=None, force_general: bool = False,
                 prefill_kernel: str = "tcgen05", fuse_decode_attention: bool = True):
        super().__init__(runtime, prefix, names)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = map(int, (hidden_size, num_heads, num_kv_heads, head_dim))
        self.qk_norm, self.qk_norm_eps, self.window = bool(qk_norm), float(qk_norm_eps), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.force_general = bool(force_general) or runtime.plain_kernels   # always use the general kernel
        if prefill_kernel not in ("tcgen05", "mma"):
            raise ValueError("prefill_kernel must be 'tcgen05' or 'mma'")
        self.prefill_kernel = prefill_kernel         # which tensor-core kernel runs prompt portions
        self.fuse_decode_attention = bool(fuse_decode_attention)   # decode-only steps: norm, rotation, cache write and
                                                                   # attention in one kernel (else three kernels)
        self.position = position            # a RotaryEmbedding part or None
        if self.position is not None and self.position.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim exceeds head_dim")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---- declarations ----
    def cache_spec(self) -> CacheSpec:
        return CacheSpec.keys_and_values(self.num_kv_heads, self.head_dim, self.window)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, KV, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        specs = {
            self.full_name("q_proj.weight"): WeightSpec((H * hd, D)),
            self.full_name("k_proj.weight"): WeightSpec((KV * hd, D)),
            self.full_name("v_proj.weight"): WeightSpec((KV * hd, D)),
            self.full_name("o_proj.weight"): WeightSpec((D, H * hd)),
        }
        if self.qk_norm:
            specs[self.full_name("q_norm.weight")] = WeightSpec((hd,), role="vector", init="norm")
            specs[self.full_name("k_norm.weight")] = WeightSpec((hd,), role="vector", init="norm")
        return specs

    def bind(self, tensors) -> None:
        parts = [tensors[self.full_name(n)] for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.float() for p in parts]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[self.full_name("o_proj.weight")]
        if self.qk_norm:
            self.q_norm_w = tensors[self.full_name("q_norm.weight")]
            self.k_norm_w = tensors[self.full_name("k_norm.weight")]

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o, self.q_norm_w, self.k_norm_w) if w is not None)

    def scratch_floats(self) -> int:
        """Upper bound of the split-KV scratch: requests * kv heads * splits never exceeds the larger of the block
        target and requests * kv heads (one split), each with 16 rows of head_dim + 2 floats."""
        most = max(self.DECODE_TARGET_BLOCKS, self.rt.workspace.max_seqs * self.num_kv_heads)
        return most * 16 * (self.head_dim + 2)

    # ---- step ----
    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = self._project(x, self.w_qkv, self.rt.workspace.rows("attn_qkv", T, (H + 2 * KV) * hd, x.dtype), T)
        return self._after_projection(qkv, ctx, cache)

    def can_fuse_norm(self, norm, ctx) -> bool:
        """A step of a few tokens can take the preceding RMSNorm (and the residual add before it) into the
        projection's weight-streaming kernel."""
        return (not self.rt.plain_kernels and getattr(norm, "weight", None) is not None and hasattr(norm, "eps")
                and ops.gemv_supported(self.rt.dtype, self.w_qkv, ctx.num_tokens)
                and not ops.gemv_splitk_preferred(self.rt.dtype, self.w_qkv, ctx.num_tokens)
                and ops.gemv_supported(self.rt.dtype, self.w_o, ctx.num_tokens))

    def forward_fused(self, h, pending, norm, ctx, cache, state, h_out):
        """h: residual stream, pending: delta not yet added (or None), h_out: where rnd(h + pending) goes (a buffer
        other than h; None without pending).  Returns (output, residual stream); the output is None when the part has
        added it to the residual stream itself (the O product's store does, where that product is the decode chain's)."""
        T = ctx.num_tokens
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        ws = self.rt.workspace
        h_new = h_out if pending is not None else h
        product = ops.gemv_stream_bf16 if ops.gemv_stream_supported(h.dtype, self.w_qkv, T) else ops.gemv_bf16
        # the O product starts behind the attention kernel; its weights are asked into the L2 from here, ahead of it
        extra = {"prefetch": self.w_o} if product is ops.gemv_stream_bf16 and self.w_o.dtype == torch.bfloat16 else {}
        qkv = product(ws.rows("attn_qkv", T, (H + 2 * KV) * hd, h.dtype), h, self.w_qkv, T, norm_weight=norm.weight,
                      eps=norm.eps, delta=pending, resid_out=h_new if pending is not None else None, **extra)
        return self._after_projection(qkv, ctx, cache, add_to=h_new), h_new

    def _after_projection(self, qkv, ctx, cache, add_to=None):
        T = qkv.shape[0]
        x = qkv
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        ws = self.rt.workspace
        g = ctx.groups[cache.group]
        pos = self.position
        att = ws.rows("attn_out", T, H * hd, x.dtype)
        if self._decode_from_projection(ctx, cache, g):
            # single decoded tokens only: per-head norm, rotation, cache write and attention in one kernel
            S = ctx.num_seqs
            splits = self.decode_splits(S, ctx.max_kv_len)
            scratch = None
            if splits > ops.DECODE_CLUSTER_SPLITS:
                scratch = ws.flat("attn_decode_scratch", self.scratch_floats(), torch.float32)
            ops.attn_decode_fused_bf16(att, qkv, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, g.slot_mapping,
                                       S, H, KV, hd, g.page_size, self.scale, splits, scratch, self.q_norm_w, self.k_norm_w,
                                       self.qk_norm_eps, pos.cos if pos is not None else None,
                                       pos.sin if pos is not None else None, window=self.window)
        else:
            q = ws.rows("attn_q", T, H * hd, x.dtype)
            ops.qk_norm_rope_kv(
                q, qkv, self.q_norm_w, self.k_norm_w,
                pos.cos if pos is not None else None, pos.sin if pos is not None else None, ctx.positions,
                g.slot_mapping if cache.writes else None, cache.pages if cache.writes else None,
                H, KV, hd, g.page_size, self.qk_norm_eps,
                rotary_dim=pos.rotary_dim if pos is not None else 0,
                interleaved=pos.interleaved if pos is not None else False)
            self.attend(att, q, ctx, cache, g)
        # Behind the attention kernel the product starts only when that kernel has ended: measured, blocks of the product
        # that arrive among the attention kernel's last blocks cost more (4 us a layer) than their early weights save.
        if add_to is not None and not self.rt.plain_kernels and ops.gemv_stream_supported(x.dtype, self.w_o, T):
            ops.gemv_stream_bf16(add_to, att, self.w_o, T, dependent=False, add_to=add_to)    # h <- rnd(h + rnd(att Wo^T)), in place
            return None
        return self._project(att, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T, dependent=False)

    def _project(self, x, w, out, rows, dependent=True):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows, dependent=dependent)

    def _decode_from_projection(self, ctx, cache, g) -> bool:
        pos = self.position
        return (ctx.all_decode and cache.writes and not self.force_general and self.fuse_decode_attention
                and ops.fast_attention_supported(self.rt.dtype, self.num_heads, self.num_kv_heads, self.head_dim, g.page_size)
                and (pos is None or (pos.rotary_dim == self.head_dim and not pos.interleaved)))

    # The split-KV decode kernel wants about two blocks per SM of a B200 and a power of two of splits: the splits of a
    # (request, kv head) are one thread-block cluster, and clusters of 5, 6, 7, 9 or 12 blocks pack badly into a GPC's SMs
    # (measured at 4,096 keys: batch 4 takes 24.5 us with 9 splits and 15.7 us with 8; batch 6 31.6 us with 6, 21.2 us with
    # 4).  Clusters of 16 blocks fit one to a GPC, so they are taken only while all of them are resident at once.
    DECODE_TARGET_BLOCKS = 296
    MAX_SPLITS = 16
    WIDE_CLUSTER_BLOCKS = 128

    def decode_splits(self, num_seqs: int, max_kv_len: int) -> int:
        pairs = max(1, num_seqs * self.num_kv_heads)
        tiles = (max_kv_len + 63) // 64
        splits = 1
        while splits * 2 <= min(self.MAX_SPLITS, tiles) and pairs * splits * 2 <= self.DECODE_TARGET_BLOCKS:
            splits *= 2
        if splits == 16 and pairs * 16 > self.WIDE_CLUSTER_BLOCKS:
            splits = 8
        return splits

    def attend(self, att, q, ctx, cache, g):
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if not self.force_general and ops.fast_attention_supported(q.dtype, H, KV, hd, g.page_size):
            S = ctx.num_seqs
            q_lens = ctx.q_lens if ctx.q_lens is not None else [1] * S
            if self.prefill_kernel == "tcgen05":
                tiles = ops.prefill_tiles_tcgen05(q_lens, H, KV)
                if tiles:
                    pieces = ops.prefill_pieces_tcgen05(tiles, KV, ctx.max_kv_len)
                    # Scratch for the pieces of long query blocks: a grid that is cut has at most one block per SM after
                    # the cut.  Made at the first prompt portion, whether that one is cut or not, so that a later
                    # capture of a graph finds it.
                    ws = self.rt.workspace
                    scratch = ws.flat("attn_prefill_pieces", ops.PREFILL_SMS * 2 * (hd + 2) * 128, torch.float32)
                    counters = ws.flat("attn_prefill_piece_counts", ops.PREFILL_SMS, torch.int32)
                    ops.attn_prefill_tcgen05(att, q, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, S, tiles,
                                             H, KV, hd, g.page_size, self.scale, window=self.window, skip_single=True,
                                             pieces=pieces, scratch=scratch, piece_counts=counters)
            else:
                tiles = ops.prefill_tiles(q_lens, H, KV)
                if tiles:
                    ops.attn_prefill_bf16(att, q, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, S, tiles,
                                          H, KV, hd, g.page_size, self.scale, window=self.window, skip_single=True)
            if any(n == 1 for n in q_lens):
                splits = self.decode_splits(S, ctx.max_kv_len)
                scratch = None
                if splits > 1:
                    n = ops.attn_decode_scratch_floats(S, KV, hd, splits)
                    scratch = self.rt.workspace.flat("attn_decode_scratch", self.scratch_floats(), torch.float32)
                    assert n <= scratch.numel()
                ops.attn_decode_bf16(att, q, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, S, H, KV, hd,
                                     g.page_size, self.scale, splits, scratch, window=self.window)
            return
        ops.paged_attention_general(att, q, cache.pages, g.block_tables, ctx.seq_of_token, ctx.positions,
                                    self.num_heads, self.num_kv_heads, self.head_dim, g.page_size, self.scale,
                                    window=self.window, num_tokens=ctx.num_tokens)
