"""Dense gated feed-forward (reference model/model_architecture.cpp:106-112,182-185; kernels/fused_ops.cu:210-220):
gu = x Wgu^T with Wgu = rows(gate_proj) over rows(up_proj); act = T( rnd(silu(g)) * u ); y = act Wdown^T; no biases."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import FeedForward, WeightSpec, register_part


@register_part("ffn", "swiglu")
class SwiGLUMLP(FeedForward):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, intermediate_size: int):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, I = self.hidden_size, self.intermediate_size
        return {
            self.full_name("gate_proj.weight"): WeightSpec((I, D)),
            self.full_name("up_proj.weight"): WeightSpec((I, D)),
            self.full_name("down_proj.weight"): WeightSpec((D, I)),
        }

    def bind(self, tensors) -> None:
        g, u = tensors[self.full_name("gate_proj.weight")], tensors[self.full_name("up_proj.weight")]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[self.full_name("down_proj.weight")]

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, x, ctx):
        T = x.shape[0]
        ws = self.rt.workspace
        act = ws.rows("ffn_act", T, self.intermediate_size, x.dtype)
        if not self.rt.plain_kernels and ops.gated_product_fused(x.dtype, self.w_gate_up, T):
            ops.gemm_bf16_tcgen05(act, x, self.w_gate_up, swiglu=True)       # gate and up never travel through memory
        else:
            gu = self._project(x, self.w_gate_up, ws.rows("ffn_gate_up", T, 2 * self.intermediate_size, x.dtype), T)
            ops.swiglu(act, gu)
        return self._down(act, T)

    def _down(self, act, T):
        return self._project(act, self.w_down, self.rt.workspace.rows("ffn_out", T, self.hidden_size, act.dtype), T)

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def can_fuse_norm(self, norm, ctx) -> bool:
        return (not self.rt.plain_kernels and getattr(norm, "weight", None) is not None and hasattr(norm, "eps")
                and ops.gemv_supported(self.rt.dtype, self.w_gate_up, ctx.num_tokens)
                and not ops.gemv_splitk_preferred(self.rt.dtype, self.w_gate_up, ctx.num_tokens)
                and ops.gemv_supported(self.rt.dtype, self.w_down, ctx.num_tokens))

    def forward_fused(self, h, pending, norm, ctx, h_out):
        """Residual add, RMSNorm, gate/up product and SwiGLU in one kernel, then the down product.  h_out: where
        rnd(h + pending) goes (a buffer other than h; unused when pending is None: the part before has added its output
        already).  Returns (output, residual stream); the output is None when the down product's store has added it to the
        residual stream itself."""
        T = ctx.num_tokens
        ws = self.rt.workspace
        h_new = h_out if pending is not None else h
        product = ops.gemv_stream_bf16 if ops.gemv_stream_supported(h.dtype, self.w_gate_up, T, swiglu=True) else ops.gemv_bf16
        act = product(ws.rows("ffn_act", T, self.intermediate_size, h.dtype), h, self.w_gate_up, T,
                      norm_weight=norm.weight, eps=norm.eps, delta=pending,
                      resid_out=h_new if pending is not None else None, swiglu=True)
        if ops.gemv_stream_supported(act.dtype, self.w_down, T):
            ops.gemv_stream_bf16(h_new, act, self.w_down, T, add_to=h_new)              # h <- rnd(h + rnd(act Wdown^T)), in place
            return None, h_new
        return self._down(act, T), h_new
