"""RMSNorm: y = x * w / sqrt(mean(x^2) + eps), computed in 32-bit
(src/kernel/core/cpu.zig:38-48,73-110).  The weight multiplies directly (no 1 + w)
and eps is added to the mean inside the root.  ``one_plus``: the stored weight lies around zero and the
multiplier is 1 + w (formed once, in 32-bit, when the weights are bound)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, TensorSpec


class RMSNorm(Norm):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.tensor = str(params.get("tensor", "weight"))   # the weight's name relative to the part
        self.one_plus = bool(params.get("one_plus", False))
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return {self.tensor: TensorSpec((self.size,), init="around_zero" if self.one_plus else "norm")}

    def bind(self, tensors):
        # norm vectors are widened to 32-bit once, as the reference does
        # (src/model/runtime/optimized_decoder/support.zig:6-19)
        self.weight = tensors[self.tensor].to(torch.float32).contiguous()
        if self.one_plus:
            self.weight = (1.0 + self.weight).contiguous()

    def forward(self, h, delta, rows=None, bias=None):
        """Adds ``delta`` (and ``bias``) into the residual ``h`` in place, then norms (the picked rows)."""
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self.ctx.dtype, rows=rows, bias=bias)
