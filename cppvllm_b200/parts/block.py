"""Pre-norm decoder block (reference model/model_architecture.cpp:150-188):

    h <- h + mixer(norm_m(h));   h <- h + ffn(norm_f(h))

The reference fuses every residual add with the norm that follows it (kernels/fused_ops.cu:70-87,
model_architecture.cpp:180,187).  The block keeps that fusion without knowing its neighbours: it receives the
residual stream `h` together with a `pending` delta that has not been added yet, folds it into its first
norm, and hands its own feed-forward output on as the next pending delta."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Block, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm, fuse_decode: bool = False):
        super().__init__(runtime, prefix, names)
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm
        self.fuse_decode = fuse_decode

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def _fused_decode(self, ctx, cache) -> bool:
        """With `fuse_decode`, a step of a few tokens through an attention mixer and a gated feed-forward runs as two
        persistent kernels around the attention (csrc/decode_fused.cu) when the parts are of the kinds those kernels
        were written for.  Off by default: at the sizes measured (hidden 1024, 8 rows) the two kernels take 33 us a
        layer where the separate kernels take 31 us; the grid barriers cost what the launches they replace cost."""
        m, f = self.mixer, self.ffn
        if not (hasattr(m, "can_fuse_decode_head") and hasattr(f, "w_gate_up") and hasattr(f, "w_down")):
            return False
        if getattr(self.ffn_norm, "weight", None) is None or not hasattr(self.ffn_norm, "eps"):
            return False
        if f.w_gate_up.dtype != torch.bfloat16 or f.w_down.dtype != torch.bfloat16:
            return False
        widths = (m.hidden_size, m.num_heads * m.head_dim, f.intermediate_size)
        return (m.can_fuse_decode_head(self.mixer_norm, ctx, cache)
                and ops.decode_fusion_supported(self.rt.dtype, ctx.num_tokens, widths, m.head_dim))

    def forward(self, h, pending, ctx, cache, state):
        if self.fuse_decode and self._fused_decode(ctx, cache):
            T = ctx.num_tokens
            ws = self.rt.workspace
            att, h = self.mixer.decode_head(h, pending, self.mixer_norm, ctx, cache)
            D, I = h.shape[1], self.ffn.intermediate_size
            h_new = ws.rows("residual_alt" if h.data_ptr() == ws.rows("residual", T, D, h.dtype).data_ptr() else "residual",
                            T, D, h.dtype)
            y2 = ws.rows("ffn_out", T, D, h.dtype)
            ops.decode_block_tail(att, self.mixer.w_o, ws.rows("attn_proj", T, D, h.dtype), h, h_new, self.ffn_norm.weight,
                                  self.ffn_norm.eps, self.ffn.w_gate_up, ws.rows("ffn_act", T, I, h.dtype), self.ffn.w_down, y2,
                                  T, ws.flat("grid_barrier", 2, torch.int32, zero=True))
            return h_new, y2
        # A part may offer to take the norm in front of it (and the residual add in front of that) into its own
        # first kernel; it says so with can_fuse_norm(norm, ctx) and then runs forward_fused.
        fuse = getattr(self.mixer, "can_fuse_norm", None)
        if fuse is not None and fuse(self.mixer_norm, ctx):
            a, h = self.mixer.forward_fused(h, pending, self.mixer_norm, ctx, cache, state)
        else:
            x = self.mixer_norm.forward(h) if pending is None else self.mixer_norm.add_forward(h, pending)
            a = self.mixer.forward(x, ctx, cache, state)
        fuse = getattr(self.ffn, "can_fuse_norm", None)
        if fuse is not None and fuse(self.ffn_norm, ctx):
            m, h = self.ffn.forward_fused(h, a, self.ffn_norm, ctx)
        else:
            x = self.ffn_norm.add_forward(h, a)
            m = self.ffn.forward(x, ctx)
        return h, m
