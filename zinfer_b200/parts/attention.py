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

Options whose changes span the whole projection row or the score (they switch the mixer to the "rows" form: one
product [q | k | v | gate] with 32-bit results, one kernel that finishes the row, the attention with the score's
changes, the gate, the output projection): ``bias`` adds a bias to q, k, v and the output projection (tensors named
like the matrices plus ``.b``; the output's is handed to the block as ``output_bias`` and joins the residual sum);
``whole_norm_eps`` norms ALL of q and all of k by their root mean square before the heads are split, with a weight
per element (``q_norm``, ``k_norm`` of the projections' sizes); ``softcap`` c caps the scaled score, s <- c tanh(s / c);
``learned_sink`` adds exp(sink[h]) to head h's denominator (tensor ``sink`` [heads]); ``distance_bias`` {rows, far,
name} adds table[bucket(i - j), h] to the capped score, where the table has ``rows`` rows (None: as many as the file's
tensor has), bucket(n) = n below rows/2
and min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2))) from there (the buckets of
"Exploring the Limits of Transfer Learning with a Unified Text-to-Text Transformer", Raffel et al., 2020, for one
direction); ``output_gate`` multiplies the heads' outputs by sigmoid(W_g x) before the output projection, ``channel``
with one gate value per output channel, ``head`` with one per head (tensor ``g``).
"""
from __future__ import annotations

import math

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
        # ---- the rows form
        self.has_bias = bool(params.get("bias", False))
        wn = params.get("whole_norm_eps")
        self.whole_norm_eps = None if wn is None else float(wn)
        self.softcap = float(params.get("softcap") or 0.0)
        self.learned_sink = bool(params.get("learned_sink", False))
        self.distance_bias = dict(params["distance_bias"]) if params.get("distance_bias") else None
        self.output_gate = params.get("output_gate")
        if self.output_gate not in (None, "channel", "head"):
            raise ValueError(f"an output gate is per channel or per head, not {self.output_gate!r}")
        self.rows_form = bool(self.has_bias or self.whole_norm_eps is not None or self.softcap or self.learned_sink
                              or self.distance_bias or self.output_gate)
        if self.rows_form:
            if self.qk_norm_eps is not None or self.values_from_keys or self.keep_first or not self.projects_kv or self.sink:
                raise ValueError("the rows form of attention goes with none of: per-head q/k norm, values from the keys, "
                                 "kept first tokens, another layer's cache, a counted sink")
            if getattr(self.position, "pairing", "halves") != "halves":
                raise ValueError("this mixer rotates pairs (i, i + dims/2) only")
            if self.distance_bias and not float(self.distance_bias["far"]) > 1.0:
                raise ValueError(f"a distance table's far end must lie beyond one token, got {self.distance_bias['far']}")
            self.n_gate = {None: 0, "channel": self.nq * self.dv, "head": self.nq}[self.output_gate]
            names.setdefault("g", "g")
            names.setdefault("sink", "sink")
            if self.whole_norm_eps is not None and "q_norm" not in (params.get("names") or {}):
                names["q_norm"], names["k_norm"] = names["q"] + ".norm", names["k"] + ".norm"
        self.output_bias = None
        self.row_bias = self.sink_logit = self.dist_table = self.w_rows = None

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
        if self.rows_form:
            if self.has_bias:
                specs[n["q"] + ".b"] = TensorSpec((q,), init="around_zero")
                specs[n["k"] + ".b"] = TensorSpec((kv,), init="around_zero")
                specs[n["v"] + ".b"] = TensorSpec((self.nkv * self.dv,), init="around_zero")
                specs[n["o"] + ".b"] = TensorSpec((self.hidden,), init="around_zero")
            if self.whole_norm_eps is not None:
                specs[n["q_norm"]] = TensorSpec((q,), init="norm")
                specs[n["k_norm"]] = TensorSpec((kv,), init="norm")
            if self.learned_sink:
                specs[n["sink"]] = TensorSpec((self.nq,), init="around_zero")
            if self.distance_bias:
                # ``rows`` None: the file gives the number of rows (random weights: as many as the far end allows, up to 32)
                free = min(32, max(2, 2 * (math.ceil(float(self.distance_bias["far"])) - 1)))
                specs[str(self.distance_bias.get("name", "rel"))] = TensorSpec((int(self.distance_bias.get("rows") or -1), self.nq),
                                                                               init="around_zero", free=free)
            if self.output_gate:
                specs[n["g"]] = TensorSpec((self.n_gate, self.hidden))
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
        if self.rows_form:
            self._bind_rows(tensors, parts)

    def _bind_rows(self, tensors, parts):
        n = self.names
        f32 = lambda t: t.to(torch.float32).contiguous()
        if self.output_gate:
            g = tensors[n["g"]]
            parts = [p.to(torch.float32) for p in parts + [g]] if any(p.dtype != g.dtype for p in parts) else parts + [g]
        self.w_rows = torch.cat(parts, dim=0).contiguous()        # one product: q, k, v and the gate
        self.w_qkv = None
        if self.has_bias:
            dev = self.w_rows.device
            self.row_bias = torch.cat([f32(tensors[n[x] + ".b"]) for x in ("q", "k", "v")]
                                      + [torch.zeros(self.n_gate, dtype=torch.float32, device=dev)]).contiguous()
            self.output_bias = f32(tensors[n["o"] + ".b"])
        if self.whole_norm_eps is not None:
            self.q_norm, self.k_norm = f32(tensors[n["q_norm"]]), f32(tensors[n["k_norm"]])
        if self.learned_sink:
            self.sink_logit = f32(tensors[n["sink"]])
        if self.distance_bias:
            table = f32(tensors[str(self.distance_bias.get("name", "rel"))])           # [rows, heads]
            rows, far = int(table.shape[0]), float(self.distance_bias["far"])
            if rows < 2 or not far > rows // 2:
                raise ValueError(f"a distance table of {rows} rows needs its far end beyond {rows // 2}, got {far}")
            buckets = distance_buckets(rows, far)
            idx = torch.tensor(buckets, dtype=torch.long, device=table.device)
            self.dist_table = table[idx].transpose(0, 1).contiguous()                    # [heads, distances]

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

    def _forward_rows(self, x, step, cache):
        # 32-bit results of the product: the biases and the norm over the whole row meet the unrounded sums
        proj = ops.linear(x, self.w_rows, out_dtype=torch.float32)
        group = step.kv_groups[cache.group]
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        q, gate = ops.qkv_rows_prepare(proj, self.row_bias, self.nq, self.nkv, self.d, self.dv, self.n_gate, self.q_norm,
                                       self.k_norm, self.whole_norm_eps or 0.0, self.rot_dims, cos, sin, step.positions,
                                       cache.k, cache.v, group.slot_mapping, cache.page_size, self.ctx.dtype)
        heads = ops.attention(q, cache.k, cache.v, group.block_tables, step, self.nq, self.nkv, self.d, cache.page_size,
                              self.window, self.scale, value_dim=self.dv, sink_logit=self.sink_logit, softcap=self.softcap,
                              dist_bias=self.dist_table)
        if gate is not None:
            heads = ops.sigmoid_gate(heads, gate, out=heads, group=self.dv if self.output_gate == "head" else 1)
        return ops.linear(heads, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)

    def forward(self, x, step, cache):
        if self.rows_form:
            if not cache.writes:
                raise ValueError("the rows form of attention fills its own cache")
            return self._forward_rows(x, step, cache)
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


def distance_buckets(rows: int, far: float) -> list[int]:
    """Row of a distance table for a key n tokens back, n = 0 .. : one token per row below rows/2, logarithmic steps up
    to ``far`` from there, the last row beyond; the list ends with the first distance that reaches the last row (every
    longer distance shares it).  Worked out in 64-bit on the host, once."""
    half = rows // 2
    out = []
    n = 0
    while True:
        b = n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b == rows - 1 and n >= half:
            return out
        n += 1
