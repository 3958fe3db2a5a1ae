"""Rotary position encoding, rotate-half pairing (i, i + d/2) over the whole head
(src/kernel/attention/rope.zig:67-90).  The part owns the cos/sin table, built on
the device by the reference's 32-bit recipe (rope.zig:25-35); equal parts share
one table.  ``scaling_factor`` f (linear scaling) divides every frequency by f: the angles are those of
position / f.  ``head_dim`` is the number of dimensions the rotation turns, which a mixer may make
smaller than its heads.

``scaling`` rescales the frequencies f_i = theta^(-2i/d) one by one (the table is then made from the
frequencies, which are worked out on the host in 64-bit and rounded once):

* ``{"kind": "by_wavelength", "factor", "low", "high", "original"}`` (the rule of the Llama 3.1 models): with the
  wavelength l = 2 pi / f, f stays where l < original/high, becomes f / factor where l > original/low, and in
  between (1 - s) f / factor + s f with s = (original/l - low) / (high - low).
* ``{"kind": "ramp", "factor", "original", "fast", "slow"}`` (YaRN: "YaRN: Efficient Context Window Extension of
  Large Language Models", Peng et al., 2023): with where(t) = d ln(original / (2 pi t)) / (2 ln theta),
  lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), d - 1) and ramp_i = clamp((i - lo) / max(hi - lo,
  0.001), 0, 1), the frequency is f_i / factor * ramp_i + f_i (1 - ramp_i); cos and sin are both multiplied by
  0.1 ln(factor) + 1.

``pairing``: ``halves`` pairs dimension i with i + d/2, ``neighbours`` 2i with 2i + 1; the table is the same, the
mixer's kernel reads the pairs accordingly (a mixer that cannot refuses)."""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding


def scaled_frequencies(head_dim: int, theta: float, scaling: dict) -> tuple[list[float], float]:
    """(frequencies, magnitude of cos and sin) under ``scaling`` (see the module's text)."""
    base = [float(theta) ** (-2.0 * i / head_dim) for i in range(head_dim // 2)]
    kind = scaling.get("kind")
    if kind == "by_wavelength":
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for f in base:
            wl = 2.0 * math.pi / f
            if wl < orig / high:
                out.append(f)
            elif wl > orig / low:
                out.append(f / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        return out, 1.0
    if kind == "ramp":
        factor, orig, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
        where = lambda turns: head_dim * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
        lo = max(math.floor(where(fast)), 0)
        hi = min(math.ceil(where(slow)), head_dim - 1)
        out = []
        for i, f in enumerate(base):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return out, 0.1 * math.log(factor) + 1.0
    raise ValueError(f"rotary scaling of kind {kind!r} is not built (by_wavelength and ramp are)")


class RotaryPosition(PositionEncoding):
    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.head_dim = int(params["head_dim"])
        self.theta = float(params["theta"])
        self.factor = float(params.get("scaling_factor", 1.0))
        self.scaling = dict(params["scaling"]) if params.get("scaling") else None
        self.pairing = str(params.get("pairing", "halves"))
        if self.pairing not in ("halves", "neighbours"):
            raise ValueError(f"rotary pairs are halves or neighbours, not {self.pairing!r}")
        if not self.factor > 0.0:
            raise ValueError(f"the rotary scaling factor must be positive, got {self.factor}")
        if self.scaling is not None and self.factor != 1.0:
            raise ValueError("a rescaling of single frequencies and a linear scaling factor exclude each other")
        if self.head_dim % 2:
            raise ValueError(f"rotary positions need an even head_dim, got {self.head_dim}")
        if self.scaling is not None:
            self.frequencies, self.magnitude = scaled_frequencies(self.head_dim, self.theta, self.scaling)
        # a request is never longer than the engine's limit nor than the model's own
        self.n_positions = min(int(params["max_positions"]), ctx.max_positions)
        self._key = ("rope", self.head_dim, self.theta, self.n_positions, self.factor,
                     tuple(sorted(self.scaling.items())) if self.scaling else None)

    def tables(self):
        """cos and sin [positions, d/2], built on the device at first use."""
        shared = self.ctx.shared
        if self._key not in shared:
            if self.scaling is not None:
                freqs = torch.tensor(self.frequencies, dtype=torch.float64).to(torch.float32).to(self.ctx.device)
                shared[self._key] = ops.rope_table_freqs(self.n_positions, freqs, self.magnitude)
            else:
                shared[self._key] = ops.rope_table(self.n_positions, self.head_dim, self.theta, self.ctx.device, self.factor)
        return shared[self._key]


class NoPosition(PositionEncoding):
    """A mixer without position encoding."""

    n_positions = None

    def tables(self):
        return None, None
