"""Grouped-query attention over the paged cache.

q = Wq x, k = Wk x, v = Wv x (one fused product); optional RMSNorm of every q and k
head with a shared [d] weight, before the position encoding; k (normed, rotated)
and v (raw) go into the request's pages; every query reads the keys at or before
its position (within ``window`` if one is set); softmax of dot * 1/sqrt(d) in
32-bit; output projection.  Query head h reads kv head h // (num_heads/num_kv_heads).
(src/model/runtime/optimized_decoder/layer.zig:110-142,188;
src/model/layers/gqa_attention/spec.zig:3-26; src/kernel/attention/basic.zig:27-76.)
The head size is independent of the model width.

Options beyond that form (each switches the mixer to the general kernels; all default to the form above):
``scale`` replaces 1/sqrt(d); ``sink`` s counts s keys of score 0 without a value in the softmax's denominator
(p_j = exp(s_j) / (s + sum exp)); ``values: "keys"`` has no value projection, a token's value is its key as
projected, before norm and rotation; a position part whose ``head_dim`` is smaller than the head rotates only
the head's first dimensions; ``names`` gives the tensors' names (q, k, v, o, q_norm, k_norm); ``keep_first`` n makes a
window keep a request's first n tokens visible (query i sees key j <= i if i - j < window or j < n; the kept tokens
keep their true positions); ``value_dim`` gives values another size than keys; ``projects_kv: False`` is a mixer
without key and value projections, which only reads a cache that another layer's run of the same head layout writes
(with its own queries, window and scale).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .base import KVCacheNeed, Mixer, TensorSpec, make_part


class GQAttention(Mixer):
    graph_safe = True   # forward() only launches kernels on device arrays: a decode step can be captured

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.nq = int(params["num_heads"])
        self.nkv = int(params["num_kv_heads"])
        self.d = int(params["head_dim"])
        if self.nkv <= 0 or self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads do not divide into {self.nkv} kv heads")
        eps = params.get("qk_norm_eps")
        self.qk_norm_eps = None if eps is None else float(eps)
        self.window = params.get("window")
        self.position = make_part(params["position"], ctx) if params.get("position") is not None else None
        # 1/sqrt(d) as a 32-bit value, applied to the score after the dot (basic.zig:50)
        self.scale = float(np.float32(1.0) / np.sqrt(np.float32(self.d)))
        if params.get("scale") is not None:
            self.scale = float(params["scale"])
        self.sink = float(params.get("sink", 0.0))
        self.values_from_keys = params.get("values", "projection") == "keys"
        if params.get("values", "projection") not in ("projection", "keys"):
            raise ValueError(f"values come from a projection or from the keys, not {params['values']!r}")
        self.keep_first = int(params.get("keep_first", 0) or 0)
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ValueError("kept first tokens go with a window and cannot be fewer than none")
        self.dv = int(params.get("value_dim") or self.d)
        self.projects_kv = bool(params.get("projects_kv", True))
        if self.values_from_keys and (self.dv != self.d or not self.projects_kv):
            raise ValueError("values taken from the keys have the keys' size and need the key projection")
        self.rot_dims = int(getattr(self.position, "head_dim", self.d)) if self.position is not None else 0
        if self.rot_dims > self.d:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit a head of {self.d}")
        names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                 "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}
        names.update(params.get("names") or {})
        self.names = names
        # what the fused kernels (norm + rotation of the whole head, plain softmax, values of their own) do not take
        self.general = bool(self.sink or self.values_from_keys or self.keep_first or self.dv != self.d or not self.projects_kv
                            or (self.position is not None and self.rot_dims != self.d and hasattr(self.position, "head_dim")))
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # ------------------------------------------------------------------ weights
    def tensor_specs(self):
        q, kv = self.nq * self.d, self.nkv * self.d
        n = self.names
        specs = {n["q"]: TensorSpec((q, self.hidden)), n["o"]: TensorSpec((self.hidden, self.nq * self.dv))}
        if self.projects_kv:
            specs[n["k"]] = TensorSpec((kv, self.hidden))
            if not self.values_from_keys:
                specs[n["v"]] = TensorSpec((self.nkv * self.dv, self.hidden))
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((self.d,), init="norm")
            specs[n["k_norm"]] = TensorSpec((self.d,), init="norm")
        return specs

    def bind(self, tensors):
        n = self.names
        parts = [tensors[n["q"]]]
        if self.projects_kv:
            parts += [tensors[n["k"]]] + ([] if self.values_from_keys else [tensors[n["v"]]])
        if len({p.dtype for p in parts}) > 1:
            parts = [p.to(torch.float32) for p in parts]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm = tensors[n["k_norm"]].to(torch.float32).contiguous()

    # -------------------------------------------------------------------- cache
    def cache_need(self):
        return KVCacheNeed(num_kv_heads=self.nkv, head_dim=self.d, window=self.window,
                           value_dim=self.dv if self.dv != self.d else None, keep_first=self.keep_first)

    def max_positions(self):
        return None if self.position is None else getattr(self.position, "n_positions", None)

    # ------------------------------------------------------------------ forward
    def heads_out(self, x, step, cache):
        """The attention's heads [T, num_heads * value size] before the output projection, by the general kernels."""
        q_width = self.nq * self.d
        if cache.writes and not self.projects_kv:
            raise ValueError("a mixer without key and value projections cannot be the one that fills its cache")
        w = self.w_qkv if cache.writes else self.w_qkv[:q_width]
        qkv = ops.linear(x, w, out_dtype=self.ctx.dtype)
        group = step.kv_groups[cache.group]
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        q = ops.qk_prepare(qkv, self.nq, self.nkv, self.d, self.rot_dims, self.q_norm, self.k_norm,
                           self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin, step.positions,
                           cache.k, cache.v, group.slot_mapping, cache.page_size,
                           values_from_keys=self.values_from_keys, write_kv=cache.writes, value_dim=self.dv)
        return ops.attention(q, cache.k, cache.v, group.block_tables, step, self.nq, self.nkv, self.d,
                             cache.page_size, self.window, self.scale, sink=self.sink, keep_first=self.keep_first,
                             value_dim=self.dv)

    def forward(self, x, step, cache):
        if self.general:
            return ops.linear(self.heads_out(x, step, cache), self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
        q_width = self.nq * self.d
        w = self.w_qkv if cache.writes else self.w_qkv[:q_width]  # a reader of another's cache needs q only
        qkv = ops.linear(x, w, out_dtype=self.ctx.dtype, allow_partials=True)
        group = step.kv_groups[cache.group]
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        if cache.writes and ops.decode_fused_ok(self.ctx.dtype, self.nq, self.nkv, self.d, step):
            # every request brings one token: norm, rotation, cache write and attention are one kernel
            o = ops.attention_decode_fused(
                qkv, self.nq, self.nkv, self.d, self.q_norm, self.k_norm,
                self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin, cache.k, cache.v,
                group.slot_mapping, group.block_tables, step, cache.page_size, self.window, self.scale)
            return ops.linear(o, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
        q = ops.qk_norm_rope_store(
            qkv, self.nq, self.nkv, self.d, self.q_norm, self.k_norm,
            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos, sin, step.positions,
            cache.k, cache.v, group.slot_mapping, cache.page_size, write_kv=cache.writes, out_dtype=self.ctx.dtype)
        o = ops.attention(q, cache.k, cache.v, group.block_tables, step, self.nq, self.nkv, self.d,
                          cache.page_size, self.window, self.scale)
        return ops.linear(o, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
