"""Dense gated feed-forward: down(act(gate(x)) * up(x)), act = silu (SwiGLU:
src/model/runtime/optimized_decoder/layer.zig:193-197, src/kernel/core/cpu.zig:130-147) or,
with ``activation: gelu_tanh``, the tanh form of gelu.  gate and up are stored as one matrix
[2I, H] so one product feeds both.  ``names`` gives the three tensors' names (gate, up, down)
where a model calls them otherwise.  ``activation: clamped_gated`` is down(g' sigmoid(``act_alpha`` g') (u' + 1)) with
g' = min(gate(x), ``limit``) and u' = clamp(up(x), -limit, limit)."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec


class SwiGLUMLP(FeedForward):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        self.clamped = self.activation == "clamped_gated"
        self.limit = float(params.get("limit") or 0.0)
        self.act_alpha = float(params.get("act_alpha", 1.0))
        if self.clamped and not self.limit > 0.0:
            raise ValueError("a clamped gate needs a positive limit")
        if self.activation not in ops.ACTIVATIONS and not self.clamped:
            raise ValueError(f"unknown activation {self.activation!r}")
        self.names = tuple(params.get("names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        gate, up, down = self.names
        return {
            gate: TensorSpec((self.inter, self.hidden)),
            up: TensorSpec((self.inter, self.hidden)),
            down: TensorSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors):
        g, u = tensors[self.names[0]], tensors[self.names[1]]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        # rows interleaved in blocks of 64 (gate block, up block) when the width allows it: the
        # tensor-core product can then apply the SwiGLU in its epilogue
        self.interleaved = self.inter % ops.SWIGLU_INTERLEAVE == 0 and not self.clamped
        self.w_gate_up = ops.interleave_gate_up(g, u) if self.interleaved else torch.cat([g, u], dim=0).contiguous()
        self.w_down = tensors[self.names[2]].contiguous()

    def forward(self, x):
        if self.interleaved:
            act = ops.linear_swiglu(x, self.w_gate_up, out_dtype=self.ctx.dtype, activation=self.activation)
        else:
            gu = ops.linear(x, self.w_gate_up, out_dtype=self.ctx.dtype, allow_partials=True)
            if self.clamped:
                act = ops.clamped_gate(gu, self.limit, self.act_alpha, 1.0, self.ctx.dtype)
            else:
                act = ops.swiglu(gu, out_dtype=self.ctx.dtype, activation=self.activation)
        # the product may come back as split-K partial sums; the next norm adds them with the residual
        return ops.linear(act, self.w_down, out_dtype=self.ctx.dtype, allow_partials=True)


class PlainMLP(FeedForward):
    """Dense feed-forward without a gate: down(act(up(x))), act = the square of relu (``relu2``).  ``names`` gives the
    two tensors' names (up, down)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "relu2"))
        if self.activation != "relu2":
            raise ValueError(f"an ungated feed-forward with activation {self.activation!r} is not built (relu2 is)")
        self.names = tuple(params.get("names", ("up", "down")))

    def tensor_specs(self):
        up, down = self.names
        return {up: TensorSpec((self.inter, self.hidden)), down: TensorSpec((self.hidden, self.inter))}

    def bind(self, tensors):
        self.w_up = tensors[self.names[0]].contiguous()
        self.w_down = tensors[self.names[1]].contiguous()

    def forward(self, x):
        mid = ops.linear(x, self.w_up, out_dtype=self.ctx.dtype, relu2=True)
        return ops.linear(mid, self.w_down, out_dtype=self.ctx.dtype, allow_partials=True)
