"""Pre-norm decoder block (reference model/model_architecture.cpp:150-188):

    h <- h + mixer(norm_m(h));   h <- h + ffn(norm_f(h))

The reference fuses every residual add with the norm that follows it (kernels/fused_ops.cu:70-87,
model_architecture.cpp:180,187).  The block keeps that fusion without knowing its neighbours: it receives the
residual stream `h` together with a `pending` delta that has not been added yet, folds it into its first
norm, and hands its own feed-forward output on as the next pending delta."""
from __future__ import annotations


from ..csrc import ops
from .base import Block, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm):
        super().__init__(runtime, prefix, names)
        self.mixer, self.ffn, self.mixer_norm, self.ffn_norm = mixer, ffn, mixer_norm, ffn_norm

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def forward(self, h, pending, ctx, cache, state):
        # A part may offer to take the norm in front of it (and the residual add in front of that) into its own
        # first kernel; it says so with can_fuse_norm(norm, ctx) and then runs forward_fused.
        # forward_fused(h, pending, norm, ..., h_out): if `pending` is not None the part writes rnd(h + pending) to h_out
        # (a buffer other than h, which the block chooses) and returns it as the residual stream beside its output.  A
        # part may return None as its output: it has then added the output to the residual stream itself.
        ws = self.rt.workspace
        T, D = ctx.num_tokens, h.shape[1]
        fuse = getattr(self.mixer, "can_fuse_norm", None)
        if fuse is not None and fuse(self.mixer_norm, ctx):
            h_out = ws.other_of_pair("residual", h, T, D, h.dtype) if pending is not None else None
            a, h = self.mixer.forward_fused(h, pending, self.mixer_norm, ctx, cache, state, h_out)
        else:
            x = self.mixer_norm.forward(h) if pending is None else self.mixer_norm.add_forward(h, pending)
            a = self.mixer.forward(x, ctx, cache, state)
        fuse = getattr(self.ffn, "can_fuse_norm", None)
        if fuse is not None and fuse(self.ffn_norm, ctx):
            m, h = self.ffn.forward_fused(h, a, self.ffn_norm, ctx, ws.other_of_pair("residual", h, T, D, h.dtype) if a is not None else None)
        else:
            x = self.ffn_norm.add_forward(h, a) if a is not None else self.ffn_norm.forward(h)
            m = self.ffn.forward(x, ctx)
        return h, m
