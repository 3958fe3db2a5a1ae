"""Latent attention: keys and values of all heads are linear maps of one small latent per token
(the multi-head latent attention of "DeepSeek-V2: A Strong, Economical, and Efficient
Mixture-of-Experts Language Model", DeepSeek-AI, 2024).

From the input h:  q = W_q h, per head [``dim`` plain | ``rot_dim`` rotated];  W_dkv h gives
``kv_rank`` values, RMS-normed into the latent c, and ``rot_dim`` values that are rotated and
serve every head as the rotated key part.  Head n has the key [W_uk,n c | rotated part] and the
value W_uv,n c; its score is (q_plain . k_plain + q_rot . k_rot) * scale, causal, plain softmax.
The concatenated heads may be gated by sigmoid(W_g h); W_o follows.

Only [c | rotated key part] is cached: one row of kv_rank + rot_dim values per token, in pages of
keys only.  The attention runs in the folded form: q_lat,n = W_uk,n^T q_plain,n, so that the score
is [q_lat,n | q_rot,n] . row, the weighted sum runs over the rows' c parts, and W_uv,n is applied
to that sum: every cached row is read once for all heads, as key and as value.

Rotary positions turn the first ``rot_dims`` of the rot_dim values (pairs (i, i + rot_dims/2), or (2i, 2i + 1) when
the position part says ``pairing: neighbours``).

Options: ``q_rank`` r sends the queries through a latent of their own, q = W_uq norm(W_dq h) (tensors ``dq``,
``dq.norm``, ``uq`` instead of ``q``; the norm has a plain weight and the layer's eps); ``window`` w lets position i
see the keys i - w + 1 .. i; ``learned_sink`` adds exp(sink[n]) to head n's softmax denominator (tensor ``sink``
[heads]; it has no value).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import KVCacheNeed, Mixer, TensorSpec, make_part


class LatentAttention(Mixer):
    graph_safe = True
    PER_HEAD_TENSOR_FROM = 128     # tokens in a step from which the per-head products go to the tensor cores

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["dim"])
        self.rot_dim = int(params["rot_dim"])
        self.vdim = int(params["vdim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["norm_eps"])
        self.gated = bool(params.get("output_gate", False))
        self.window = params.get("window")
        self.q_rank = int(params.get("q_rank") or 0)
        self.learned_sink = bool(params.get("learned_sink", False))
        self.position = make_part(params["position"], ctx)
        self.neighbours = getattr(self.position, "pairing", "halves") == "neighbours"
        self.rot_dims = int(getattr(self.position, "head_dim", self.rot_dim))
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit the rotated part of {self.rot_dim}")
        self.row = self.rank + self.rot_dim          # a cached row
        if self.row > 640:
            raise ValueError(f"cached rows of {self.row} values are wider than the attention kernel takes (640)")

    # ------------------------------------------------------------------ weights
    def tensor_specs(self):
        H, hid = self.heads, self.hidden
        qw = H * (self.dim + self.rot_dim)
        queries = {"q": TensorSpec((qw, hid))} if not self.q_rank else {
            "dq": TensorSpec((self.q_rank, hid)), "dq.norm": TensorSpec((self.q_rank,), init="norm"),
            "uq": TensorSpec((qw, self.q_rank))}
        specs = {
            **queries,
            "dkv": TensorSpec((self.row, hid)),
            "dkv.norm": TensorSpec((self.rank,), init="norm"),
            "uk": TensorSpec((H * self.dim, self.rank)),
            "uv": TensorSpec((H * self.vdim, self.rank)),
            "o": TensorSpec((hid, H * self.vdim)),
        }
        if self.gated:
            specs["g"] = TensorSpec((H * self.vdim, hid))
        if self.learned_sink:
            specs["sink"] = TensorSpec((H,), init="around_zero")
        return specs

    def bind(self, tensors):
        parts = [tensors["dq" if self.q_rank else "q"], tensors["dkv"]] + ([tensors["g"]] if self.gated else [])
        if len({p.dtype for p in parts}) > 1:
            parts = [p.to(torch.float32) for p in parts]
        self.w_in = torch.cat(parts, dim=0).contiguous()      # one product: queries, latent, gate
        self.c_norm = tensors["dkv.norm"].to(torch.float32).contiguous()
        H = self.heads
        # per head the key map transposed, [rank, dim]: q_lat = q_plain @ W_uk,n
        self.w_uk_t = tensors["uk"].view(H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["uv"].view(H, self.vdim, self.rank).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.sink_logit = tensors["sink"].to(torch.float32).contiguous() if self.learned_sink else None
        if self.q_rank:
            self.q_norm = tensors["dq.norm"].to(torch.float32).contiguous()
            self.w_uq = tensors["uq"].contiguous()

    # -------------------------------------------------------------------- cache
    def cache_need(self):
        return KVCacheNeed(num_kv_heads=1, head_dim=self.row, window=self.window, values=False)

    def max_positions(self):
        return getattr(self.position, "n_positions", None)

    # ------------------------------------------------------------------ forward
    def _per_head(self, x, weight, out):
        """out[:, n] = x[:, n] @ weight[n]^T for every head n (views [T, heads, *]).  Many tokens in bfloat16: the
        tensor-core kernel's form with one product per head in one launch (or, where the views do not meet its
        rules, one launch per head); few tokens (a decode step) and float32: all heads in one launch of the
        batched CUDA-core product, which is bound by reading the weights once either way."""
        if x.shape[0] > self.PER_HEAD_TENSOR_FROM and ops.linear_heads_ok(x, weight, out):
            return ops.linear_heads(x, weight, out)       # all heads in one launch
        if x.shape[0] > self.PER_HEAD_TENSOR_FROM and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 \
                and ops.tensor_core_linear_ok(x[:, 0], weight[0]) and ops.tensor_core_linear_ok(x[:, -1], weight[-1]):
            for n in range(self.heads):
                ops.linear(x[:, n], weight[n], out=out[:, n])
        else:
            ops.linear_batched(x.transpose(0, 1), weight, out.transpose(0, 1))
        return out

    def forward(self, x, step, cache):
        T, H, D = x.shape[0], self.heads, self.row
        qw = H * (self.dim + self.rot_dim)
        group = step.kv_groups[cache.group]
        cos, sin = self.position.tables()
        q_eff = torch.empty((T, H, D), dtype=self.ctx.dtype, device=x.device)
        if self.q_rank:
            # queries through their own latent: [W_dq; W_dkv; W_g] h with 32-bit results (both norms meet the unrounded
            # sums), the norm of the query latent, W_uq
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
            qs = ops.linear(ops.rmsnorm_rows(proj[:, :self.q_rank], self.q_norm, self.eps, self.ctx.dtype), self.w_uq,
                            out_dtype=self.ctx.dtype)
            ops.latent_prepare_rows(qs, proj[:, self.q_rank:], H, self.dim, self.rot_dim, self.rank, self.rot_dims,
                                    self.neighbours, self.c_norm, self.eps, cos, sin, step.positions, q_eff,
                                    cache.k if cache.writes else None, group.slot_mapping)
            gate_at = self.q_rank + D
        else:
            proj = qs = ops.linear(x, self.w_in, out_dtype=self.ctx.dtype)
            if self.neighbours:
                ops.latent_prepare_rows(proj, proj[:, qw:], H, self.dim, self.rot_dim, self.rank, self.rot_dims, True,
                                        self.c_norm, self.eps, cos, sin, step.positions, q_eff,
                                        cache.k if cache.writes else None, group.slot_mapping)
            else:
                ops.latent_prepare(proj, H, self.dim, self.rot_dim, self.rank, self.rot_dims, self.c_norm, self.eps, cos, sin,
                                   step.positions, q_eff, cache.k if cache.writes else None, group.slot_mapping)
            gate_at = qw + D
        q_plain = qs[:, :qw].view(T, H, self.dim + self.rot_dim)[:, :, :self.dim]
        self._per_head(q_plain, self.w_uk_t, q_eff[:, :, :self.rank])
        lat = ops.latent_attention(q_eff.view(T, H * D), cache.k, group.block_tables, step, H, self.rank,
                                   cache.page_size, self.window, self.scale, sink_logit=self.sink_logit)
        heads = torch.empty((T, H, self.vdim), dtype=self.ctx.dtype, device=x.device)
        self._per_head(lat.view(T, H, self.rank), self.w_uv, heads)
        heads = heads.view(T, H * self.vdim)
        if self.gated:
            gate = proj[:, gate_at:gate_at + H * self.vdim]
            heads = ops.sigmoid_gate(heads, gate if gate.dtype == heads.dtype else gate.to(heads.dtype), out=heads)
        return ops.linear(heads, self.w_o, out_dtype=self.ctx.dtype, allow_partials=True)
