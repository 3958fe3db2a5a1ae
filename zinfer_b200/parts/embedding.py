"""Token embedding and output head
(src/model/runtime/optimized_decoder/runtime.zig:109-115,139-146)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec


class TokenEmbedding(Part):
    """h0 = table[token]; no scaling.  Gives the 32-bit residual stream."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params.get("name", "embed_tokens") + params.get("suffix", ".weight")
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors):
        self.weight = tensors[self.name].contiguous()

    def forward(self, token_ids):
        return ops.embed_gather(self.weight, token_ids)


class HashedBigramEmbedding(TokenEmbedding):
    """h0 = ``scale`` * table[token] + pairs[row], where ``row`` hashes the token and the one before it:
    (previous * ``mul_prev`` + token * ``mul_cur``) mod ``buckets``; a request's first token takes the pair table's
    last row (number ``buckets``).  ``pairs`` None leaves the second table out (a scaled embedding).

    The token before a step's first token of a request was brought by an earlier step, so the part keeps every
    request's last token as per-request state (one int32 per slot), on the device: a token that the step before
    sampled and that never reached the host is found there as well."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.scale = float(params.get("scale", 1.0))
        pairs = params.get("pairs")
        self.pairs_name = None if pairs is None else str(pairs["name"])
        self.buckets = int(pairs["buckets"]) if pairs is not None else 0
        self.mul_prev = int(pairs["mul_prev"]) if pairs is not None else 0
        self.mul_cur = int(pairs["mul_cur"]) if pairs is not None else 0
        if pairs is not None and self.buckets <= 0:
            raise ValueError(f"a table of token pairs needs at least one bucket, got {self.buckets}")
        self.pairs = None

    def tensor_specs(self):
        specs = super().tensor_specs()
        if self.pairs_name is not None:
            specs[self.pairs_name] = TensorSpec((self.buckets + 1, self.hidden))
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        if self.pairs_name is not None:
            pairs = tensors[self.pairs_name]
            if pairs.dtype != self.weight.dtype:       # one of them is stored in 32-bit: both are read as 32-bit
                pairs, self.weight = pairs.to(torch.float32), self.weight.to(torch.float32).contiguous()
            self.pairs = pairs.contiguous()

    def cache_need(self):
        from .base import StateNeed
        return StateNeed((1,), torch.int32)

    def forward(self, token_ids, step=None, state=None):
        if step is None or state is None:
            raise ValueError("an embedding that looks at the token before needs the step and its per-request state")
        return ops.embed_bigram(self.weight, self.pairs, token_ids, step, state.state, self.scale, self.buckets,
                                self.mul_prev, self.mul_cur)


class LMHead(Part):
    """logits = scale * W x in 32-bit (``scale`` 1 unless the model gives one).  ``tied_to`` names the
    embedding whose table stands for W; a separate ``<name>.weight`` in the file is then optional and unused."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.name = params.get("name", "lm_head") + params.get("suffix", ".weight")
        self.tied_to = params.get("tied_to")
        self.scale = float(params.get("scale", 1.0))
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab, self.hidden), optional=self.tied_to is not None)}

    def bind(self, tensors):
        if self.tied_to is None:
            self.weight = tensors[self.name].contiguous()

    def tie(self, table: torch.Tensor):
        self.weight = table

    def forward(self, x):
        logits = ops.linear(x, self.weight, out_dtype=torch.float32)
        return logits if self.scale == 1.0 else ops.scale_(logits, self.scale)

    def forward_argmax(self, x):
        """The logits and each row's first maximum, found in the product's own epilogue where the
        tensor-core kernel takes the shape."""
        if self.scale == 1.0:
            return ops.linear_argmax(x, self.weight)
        logits = self.forward(x)
        return logits, ops.argmax(logits)
