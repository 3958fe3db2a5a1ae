"""The pre-norm arrangement: h1 = h + mixer(norm(h)); h2 = h1 + ffn(norm(h1))
(src/model/layers/rmsnorm_gqa_swiglu_block.zig:86-88,161-163).

The residual stream ``h`` is 32-bit.  An update that has not yet been added is
carried as ``pending`` into the next norm, where the add is fused with the norm;
the block therefore returns its feed-forward's output instead of adding it.

Options: ``residual_scale`` m multiplies both updates (h + m * mixer(..), h1 + m * ffn(..));
``feed_forward`` None leaves the second half out; ``verbatim_names`` takes the four name
parameters as complete prefixes (``norm1`` for a tensor called just that) instead of
appending a dot."""
from __future__ import annotations

from .. import ops
from .base import Block, make_part, prefixed, take


class PreNormBlock(Block):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.mixer = make_part(params["mixer"], ctx)
        self.mixer_norm = make_part(params["mixer_norm"], ctx)
        has_ffn = params.get("feed_forward") is not None
        self.feed_forward = make_part(params["feed_forward"], ctx) if has_ffn else None
        # a block whose sublayers read the same norm's output names no second norm
        self.ffn_norm = make_part(params["ffn_norm"], ctx) if has_ffn and params.get("ffn_norm") is not None else None
        self.residual_scale = float(params.get("residual_scale", 1.0))
        dot = "" if params.get("verbatim_names") else "."
        self._names = {
            "mixer": params.get("mixer_name", "mixer") + dot,
            "feed_forward": params.get("ffn_name", "feed_forward") + dot,
            "mixer_norm": params.get("mixer_norm_name", "mixer_norm") + dot,
            "ffn_norm": params.get("ffn_norm_name", "ffn_norm") + dot,
        }

    def _parts(self):
        return [(self._names[k], getattr(self, k)) for k in ("mixer_norm", "mixer", "ffn_norm", "feed_forward")
                if getattr(self, k) is not None]

    def tensor_specs(self):
        out = {}
        for prefix, part in self._parts():
            out.update(prefixed(prefix, part.tensor_specs()))
        return out

    def bind(self, tensors):
        for prefix, part in self._parts():
            part.bind(take(tensors, prefix))

    def _update(self, delta):
        return delta if self.residual_scale == 1.0 else ops.Scaled(delta, self.residual_scale)

    def forward(self, h, pending, step, cache, bias=None):
        if self.feed_forward is not None and self.ffn_norm is None:
            raise ValueError("this arrangement needs a norm before its feed-forward")
        x = self.mixer_norm.forward(h, pending) if bias is None else self.mixer_norm.forward(h, pending, bias=bias)
        a = self._update(self.mixer.forward(x, step, cache))
        if getattr(self.mixer, "output_bias", None) is not None:
            a = ops.Several([a], row_bias=self.mixer.output_bias * self.residual_scale)
        if self.feed_forward is None:
            return a
        x = self.ffn_norm.forward(h, a)
        return self._update(self.feed_forward.forward(x))


class OutputNormBlock(PreNormBlock):
    """The arrangement that norms a sublayer's OUTPUT: h1 = h + norm1(mixer(h)); h2 = h1 + norm2(ffn(h1)).
    The sublayers read the residual stream itself (in the activations' type).  Same parameters and tensor
    names as :class:`PreNormBlock`; ``residual_scale`` multiplies the normed update's input, which the norm
    undoes, so it is refused unless 1.

    Nothing is left pending: the norm's kernel adds the normed output into ``h`` and hands back ``h`` in the
    activations' type, which the next sublayer (or, as :class:`ops.Carried`, the next block) reads."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        if self.residual_scale != 1.0:
            raise ValueError("a block that norms its sublayers' outputs takes no residual multiplier")

    def forward(self, h, pending, step, cache, bias=None):
        if bias is not None:
            raise ValueError("a block that norms its sublayers' outputs takes no per-pass vector")
        if isinstance(pending, ops.Carried):
            x = pending.x
        else:
            if pending is not None:
                ops.residual_add(h, pending)
            x = ops.cast_rows(h, self.ctx.dtype)
        mixed = self.mixer.forward(x, step, cache)
        a, b = mixed if isinstance(mixed, tuple) else (mixed, None)        # a mixer of two branches hands back both
        x = ops.norm_residual(h, a, self.mixer_norm.weight, self.mixer_norm.eps, self.ctx.dtype, b=b)
        if self.feed_forward is None:
            return ops.Carried(x)
        out = self.feed_forward.forward(x)
        a, b = out if isinstance(out, tuple) else (out, None)              # routed experts beside a shared one
        x = ops.norm_residual(h, a, self.ffn_norm.weight, self.ffn_norm.eps, self.ctx.dtype, b=b)
        return ops.Carried(x)


class ParallelBlock(PreNormBlock):
    """The arrangement whose two sublayers read the SAME stream: h1 = h + mixer(norm1(h)) + ffn(norm2(h)), each norm
    with its own weight.  Same parameters and tensor names as :class:`PreNormBlock`.

    Both norms share their root mean square, so one kernel makes both from one pass over the stream, and the same
    pass adds what the block before left pending.  The block leaves all its updates pending as :class:`ops.Several`
    (the mixer's output, the feed-forward's, and a shared expert's where the feed-forward hands back a pair): the
    next block's norm, or the model's last one, adds them, in this order.  Without ``ffn_norm`` both sublayers read the
    ONE norm's output, h1 = h + mixer(n) + ffn(n) with n = norm1(h).  A mixer's ``output_bias`` (a vector its output
    projection adds to every token) goes with the pending updates and is added by the same kernel."""

    def forward(self, h, pending, step, cache, bias=None):
        row_bias = getattr(self.mixer, "output_bias", None)
        if row_bias is not None and self.residual_scale != 1.0:
            row_bias = row_bias * self.residual_scale
        if self.feed_forward is None or self.ffn_norm is None:
            x1 = x2 = ops.sum_norm(h, pending, self.mixer_norm.weight, self.mixer_norm.eps, self.ctx.dtype, bias=bias)
        else:
            x1, x2 = ops.add_rmsnorm_pair(h, pending, self.mixer_norm.weight, self.ffn_norm.weight, self.mixer_norm.eps,
                                          self.ffn_norm.eps, self.ctx.dtype, bias=bias)
        a = self.mixer.forward(x1, step, cache)
        if self.feed_forward is None:
            return self._update(a) if row_bias is None else ops.Several([self._update(a)], row_bias=row_bias)
        out = self.feed_forward.forward(x2)
        return ops.Several([self._update(t) for t in (a, *(out if isinstance(out, tuple) else (out,)))], row_bias=row_bias)
