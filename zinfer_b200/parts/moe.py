"""Mixture of experts: every token runs ``top`` of ``experts`` small feed-forwards and takes the
weighted sum of their outputs.

Router: logits z = W_r h over ``experts + identity`` outputs in 32-bit, scores s = softmax(z).  A token chooses the ``top`` outputs with the largest s + correction
(a per-output vector; the selection bias of auxiliary-loss-free balancing) and weights them by
s without the correction, divided by their sum only if ``renormalize``.  The last ``identity``
outputs stand for experts without weights whose output is their input.  An expert is
W_down act(W_up h) with act the square of relu (``relu2``).

Other routers and experts, by parameter: ``score: sigmoid`` scores each output alone, s = sigmoid(z);
a ``correction`` is then added to the sigmoid scores for the choice alone, as with the softmax;
``groups`` / ``groups_kept`` cut the experts into equal groups of neighbours, score a group by the sum of its two
largest scores and let only experts of the best groups be chosen; ``weight_scale`` multiplies the weights;
``activation: silu_gated`` makes an expert W_down (silu(W_gate h) * (W_up h)); ``shared`` (a feed-forward part) runs
for every token beside the routed experts, and ``forward`` then hands back the pair (routed, shared) for the block
to add.  ``score: top_logits`` chooses the ``top`` largest logits themselves (``router_bias``: a bias ``router.b`` on the
logits) and weights them by the softmax over the chosen logits alone.  ``activation: clamped_gated`` makes an expert
W_down (g' sigmoid(``act_alpha`` g') (u' + 1)) with g' = min(W_gate h, ``limit``) and u' = clamp(W_up h, -limit, limit).

The chosen (token, expert) pairs are laid out by expert on the device, in whole tiles, and two
grouped products run over them; nothing is read back, so a decode step can be captured.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec


class RoutedExperts(FeedForward):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.experts = int(params["experts"])
        self.identity = int(params.get("identity_experts", 0))
        self.top = int(params["top"])
        self.renormalize = bool(params.get("renormalize", False))
        self.has_correction = bool(params.get("correction", False))
        act = params.get("activation", "relu2")
        if act not in ("relu2", "silu_gated", "clamped_gated"):
            raise ValueError(f"experts with activation {act!r} are not built (relu2, silu_gated and clamped_gated are)")
        self.gated = act in ("silu_gated", "clamped_gated")
        self.clamped = act == "clamped_gated"
        self.limit = float(params.get("limit") or 0.0)
        self.act_alpha = float(params.get("act_alpha", 1.0))
        if self.clamped and not self.limit > 0.0:
            raise ValueError("clamped experts need a positive limit")
        self.score = params.get("score", "softmax")
        if self.score not in ("softmax", "sigmoid", "top_logits"):
            raise ValueError(f"router scores are softmax, sigmoid or top_logits, not {self.score!r}")
        self.router_bias = bool(params.get("router_bias", False))
        if self.router_bias and self.score != "top_logits":
            raise ValueError("a bias on the router's logits is built for the choice by the logits themselves")
        self.groups = int(params.get("groups", 1))
        self.groups_kept = int(params.get("groups_kept", self.groups))
        self.weight_scale = float(params.get("weight_scale", 1.0))
        # the fused router kernel has the softmax over all outputs; everything else takes the general choice
        self.general_route = self.score != "softmax" or self.groups > 1 or self.weight_scale != 1.0
        self.top_logits = self.score == "top_logits"
        if self.top_logits:
            if self.groups > 1 or self.weight_scale != 1.0 or self.has_correction or self.identity:
                raise ValueError("the choice by the logits themselves takes no groups, scale, correction or identity experts")
        elif self.general_route:
            if self.identity:
                raise ValueError("identity experts are built for the softmax router without groups only")
            if self.groups <= 0 or self.experts % self.groups or not 1 <= self.groups_kept <= self.groups:
                raise ValueError(f"{self.experts} experts do not form {self.groups} groups of which {self.groups_kept} are kept")
            if self.top > self.groups_kept * (self.experts // self.groups):
                raise ValueError(f"{self.top} experts cannot be chosen from {self.groups_kept} groups of {self.experts // self.groups}")
        from .base import make_part
        self.shared = make_part(params["shared"], ctx) if params.get("shared") is not None else None
        self.shared_name = params.get("shared_name", "shared.")
        self.gate_name = params.get("gate_name", "gate")
        self.outputs = self.experts + self.identity
        if not 1 <= self.top <= self.outputs:
            raise ValueError(f"{self.top} of {self.outputs} router outputs cannot be chosen")
        self.expert_names = params.get("expert_names", "e{}.")     # prefix of expert i's tensors
        # from this many (token, expert) pairs in a step the products go to the tensor cores (bfloat16)
        self.tensor_core_pairs = int(params.get("tensor_core_pairs", 64))

    def tensor_specs(self):
        specs = {"router": TensorSpec((self.outputs, self.hidden))}
        if self.has_correction:
            specs["correction"] = TensorSpec((self.outputs,), init="zeros")
        if self.router_bias:
            specs["router.b"] = TensorSpec((self.outputs,), init="around_zero")
        for e in range(self.experts):
            p = self.expert_names.format(e)
            if self.gated:
                specs[p + self.gate_name] = TensorSpec((self.inter, self.hidden))
            specs[p + "up"] = TensorSpec((self.inter, self.hidden))
            specs[p + "down"] = TensorSpec((self.hidden, self.inter))
        if self.shared is not None:
            from .base import prefixed
            specs.update(prefixed(self.shared_name, self.shared.tensor_specs()))
        return specs

    def bind(self, tensors):
        self.w_router = tensors["router"].contiguous()
        self.correction = tensors["correction"].to(torch.float32).contiguous() if self.has_correction else None
        self.bias = tensors["router.b"].to(torch.float32).contiguous() if self.router_bias else None
        ups = [tensors[self.expert_names.format(e) + "up"] for e in range(self.experts)]
        if self.gated:     # an expert's gate rows above its up rows: one product feeds both
            gates = [tensors[self.expert_names.format(e) + self.gate_name] for e in range(self.experts)]
            ups = [torch.cat([g, u] if g.dtype == u.dtype else [g.to(torch.float32), u.to(torch.float32)], dim=0)
                   for g, u in zip(gates, ups)]
        if self.shared is not None:
            from .base import take
            self.shared.bind(take(tensors, self.shared_name))
        downs = [tensors[self.expert_names.format(e) + "down"] for e in range(self.experts)]
        if len({t.dtype for t in ups + downs}) > 1:
            ups, downs = [t.to(torch.float32) for t in ups], [t.to(torch.float32) for t in downs]
        dev = self.w_router.device
        self.up_rows = (2 if self.gated else 1) * self.inter
        self.w_up = torch.stack(ups).contiguous() if ups else torch.empty((0, self.up_rows, self.hidden), device=dev)
        self.w_down = torch.stack(downs).contiguous() if downs else torch.empty((0, self.hidden, self.inter), device=dev)

    def forward(self, x):
        routed = self.routed(x)
        if self.shared is None:
            return routed
        return routed, self.shared.forward(x)

    def _act(self, mid2):
        """Between an expert's two products, where the first one's kernel has not done it: the gate."""
        if self.clamped:
            return ops.clamped_gate(mid2, self.limit, self.act_alpha, 1.0, self.ctx.dtype)
        return ops.swiglu(mid2, out_dtype=self.ctx.dtype, activation="silu") if self.gated else mid2

    def routed(self, x):
        T = x.shape[0]
        relu2 = not self.gated
        if self.top_logits:
            chosen, weight = ops.moe_router_top_logits(x, self.w_router, self.bias, self.top)
        elif self.general_route and self.hidden <= 32768:
            chosen, weight = ops.moe_router_grouped(x, self.w_router, self.top, self.score, self.groups, self.groups_kept,
                                                    self.weight_scale, self.renormalize, correction=self.correction)
        elif self.general_route:
            logits = ops.linear_cuda_cores(x, self.w_router, out_dtype=torch.float32)     # 32-bit multiply-adds
            chosen, weight = ops.moe_route_grouped(logits, self.top, self.score, self.groups, self.groups_kept,
                                                   self.weight_scale, self.renormalize, correction=self.correction)
        elif self.hidden <= 32768:      # the router's product and the choice in one kernel (the row fits its shared memory)
            chosen, weight = ops.moe_router(x, self.w_router, self.correction, self.top, self.renormalize)
        else:
            logits = ops.linear_cuda_cores(x, self.w_router, out_dtype=torch.float32)     # 32-bit multiply-adds
            chosen, weight = ops.moe_route(logits, self.correction, self.top, self.renormalize)
        pairs = T * self.top
        if pairs >= self.tensor_core_pairs and x.dtype == torch.bfloat16 and self.experts > 0 \
                and ops.linear_grouped_tensor_ok(self.w_up) and ops.linear_grouped_tensor_ok(self.w_down):
            # a prompt's portion in bfloat16: the pairs' rows are gathered by expert into tiles of 128 and
            # both products run on the tensor cores
            tile = ops.MOE_TILE_ROWS_TENSOR
            row_token, row_self, pair_row, tile_expert, n_tiles = ops.moe_align(chosen, self.experts, tile)
            rows = row_token.numel()
            xs = ops.gather_rows(x, row_token)
            mid = torch.empty((rows, self.up_rows), dtype=self.ctx.dtype, device=x.device)
            ops.linear_grouped_tensor(xs, self.w_up, mid, tile_expert, relu2=relu2, pairs=pairs)
            y = torch.empty((rows, self.hidden), dtype=torch.float32, device=x.device)
            ops.linear_grouped_tensor(self._act(mid), self.w_down, y, tile_expert, pairs=pairs)
            return ops.moe_combine(y, x, chosen, weight, pair_row, self.experts)
        tile = ops.MOE_TILE_ROWS if pairs > 16 * max(self.experts, 1) else ops.MOE_TILE_ROWS_SMALL
        row_token, row_self, pair_row, tile_expert, n_tiles = ops.moe_align(chosen, self.experts, tile)
        rows = row_token.numel()
        mid = torch.empty((rows, self.up_rows), dtype=self.ctx.dtype, device=x.device)
        y = torch.empty((rows, self.hidden), dtype=torch.float32, device=x.device)
        if tile == ops.MOE_TILE_ROWS_SMALL and ops.linear_few_rows_ok(x, self.w_up) \
                and ops.linear_few_rows_ok(mid[:, :self.inter], self.w_down):
            # few rows per expert (a decode step): the experts' weights are streamed once, bound by memory
            ops.linear_few_rows(x, self.w_up, mid, row_token, tile_expert, n_tiles, relu2=relu2)
            ops.linear_few_rows(self._act(mid), self.w_down, y, row_self, tile_expert, n_tiles)
        else:
            ops.linear_grouped(x, self.w_up, mid, row_token, tile_expert, n_tiles, tile, relu2=relu2)
            ops.linear_grouped(self._act(mid), self.w_down, y, row_self, tile_expert, n_tiles, tile)
        return ops.moe_combine(y, x, chosen, weight, pair_row, self.experts)
