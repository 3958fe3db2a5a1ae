"""A plain, slow implementation of the Sepitar design in 64-bit arithmetic: the oracle of the tests.

One function per mechanism, written from the design's equations; it shares no code with the engine.
Weights come as a dictionary name -> tensor (any floating type; widened to float64), the configuration as
the dictionary of config.json.

The design in short.  A layer norms the stream once and adds both sublayers' outputs: with n = N(x),
x <- x + mixer(n) + ff(n); N is an RMS norm whose stored weight lies around zero (the multiplier is 1 + w).
Three mixers.  ``attention``: grouped queries with biases on q, k, v and o, no rotation, a learned bias per
head and distance bucket (buckets one token wide near the query, logarithmic further away), a sliding window,
a sigmoid gate per output channel.  ``attention_2``: an RMS norm over the whole of q (and of k) before the
heads are split, a rotation of each head's first dimensions in pairs (i, i + dims/2) with frequencies rescaled
by wavelength, a tanh cap on the scores, all earlier keys visible, a learned sink per head in the softmax's
denominator, a sigmoid gate per head.  ``latent_attention``: queries through a normed low-rank latent, keys and
values from one normed latent per token plus one rotated key part shared by all heads, rotation in
neighbouring pairs (2i, 2i + 1) with ramped frequency scaling and a magnitude factor, a window, a sink.  The
feed-forward is a mixture of clamped gated experts (router logits with a bias, the largest ``top`` chosen,
softmax over the chosen) beside a shared expert.  A range of layers may run several times in a row; before
every pass but the first the embedding's output is added to the stream.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
ACT_ALPHA = 1.702          # the experts' gate is g * sigmoid(ACT_ALPHA * g)


def _w(t):
    return t.to(F64)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + _w(w))


def norm_plain(x, w, eps):
    return rms(x, eps) * _w(w)


# --------------------------------------------------------------------------------- the order of layers
def layer_runs(cfg):
    """[(layer, pass number, first of its pass)] in the order in which layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, 0, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, 0, False) for i in range(a)]
    for p in range(times):
        runs += [(i, p, i == a and p > 0) for i in range(a, b)]
    return runs + [(i, 0, False) for i in range(b, n)]


# ------------------------------------------------------------------------------------------ positions
def distance_bucket(n, rows, far):
    """Row of the distance table for a key ``n`` tokens back."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def frequencies(rot):
    d = int(rot["dims"])
    return [float(rot["base"]) ** (-2.0 * i / d) for i in range(d // 2)]


def frequencies_by_wavelength(rot):
    """Frequencies kept where the wavelength is short, divided by ``factor`` where it is long, blended between."""
    s = rot["scaling"]
    out = []
    for f in frequencies(rot):
        wl = 2.0 * math.pi / f
        if wl < s["original"] / s["high"]:
            out.append(f)
        elif wl > s["original"] / s["low"]:
            out.append(f / s["factor"])
        else:
            t = (s["original"] / wl - s["low"]) / (s["high"] - s["low"])
            out.append((1.0 - t) * f / s["factor"] + t * f)
    return out


def frequencies_ramped(rot):
    """(frequencies, magnitude): a ramp over the pair index between two turn counts decides how much of the division
    by ``factor`` a pair takes; cos and sin are both multiplied by the magnitude."""
    s = rot["scaling"]
    d, base = int(rot["dims"]), float(rot["base"])
    where = lambda turns: d * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(s["fast"])), 0)
    hi = min(math.ceil(where(s["slow"])), d - 1)
    out = []
    for i, f in enumerate(frequencies(rot)):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(f / s["factor"] * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(s["factor"]) + 1.0


def rotate_half(x, positions, freqs, magnitude=1.0):
    """x [..., T, heads, d]: the first 2 * len(freqs) dimensions in pairs (i, i + n)."""
    n = len(freqs)
    a = positions.to(F64).unsqueeze(-1) * torch.tensor(freqs, dtype=F64)
    c, s = (torch.cos(a) * magnitude).unsqueeze(1), (torch.sin(a) * magnitude).unsqueeze(1)
    u, v = x[..., :n], x[..., n:2 * n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * n:]], dim=-1)


def rotate_pairs(x, positions, freqs, magnitude=1.0):
    """x [T, heads, d]: the first 2 * len(freqs) dimensions in pairs (2i, 2i + 1)."""
    n = len(freqs)
    a = positions.to(F64).unsqueeze(-1) * torch.tensor(freqs, dtype=F64)
    c, s = (torch.cos(a) * magnitude).unsqueeze(1), (torch.sin(a) * magnitude).unsqueeze(1)
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., 2 * n:]], dim=-1)


# -------------------------------------------------------------------------------------------- softmax
def attend(scores, values, visible, sink=None):
    """scores [H, T, n], values [H, n, V], visible [T, n] bool, sink [H] or None -> [T, H * V].  The sink adds
    exp(sink) to a head's denominator and nothing else."""
    s = scores.masked_fill(~visible.unsqueeze(0), -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.view(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.view(-1, 1, 1) - m)
    out = (e / den) @ values
    return out.transpose(0, 1).reshape(out.shape[1], -1)


def causal(pos, n_keys, window=None):
    j = torch.arange(n_keys).unsqueeze(0)
    i = pos.unsqueeze(1)
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    return ok


# --------------------------------------------------------------------------------------------- mixers
def attention_cache(h, p, m, pos0):
    """What the cache of an ``attention`` layer holds for the tokens h at positions pos0..: keys and values."""
    T = h.shape[0]
    k = (h @ _w(p["k"]).T + _w(p["k.b"])).view(T, m["kv_heads"], m["dim"])
    v = (h @ _w(p["v"]).T + _w(p["v.b"])).view(T, m["kv_heads"], m["vdim"])
    return k, v


def attention(h, p, m, pos0, cache):
    """``cache`` = (keys, values) of positions 0 .. pos0 + T - 1."""
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    keys, values = cache
    n = keys.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ _w(p["q"]).T + _w(p["q.b"])).view(T, H, D)
    rep = H // G
    kh = keys.repeat_interleave(rep, dim=1).permute(1, 0, 2)           # [H, n, D]
    vh = values.repeat_interleave(rep, dim=1).permute(1, 0, 2)
    scores = torch.einsum("thd,hnd->htn", q, kh) * float(m["scale"])
    rel = _w(p["rel"])
    rows = rel.shape[0]
    dist = (pos.unsqueeze(1) - torch.arange(n).unsqueeze(0)).clamp(min=0)
    bucket = torch.tensor([[distance_bucket(int(x), rows, m["bias_max"]) for x in row] for row in dist.tolist()])
    scores = scores + rel[bucket].permute(2, 0, 1)
    mask = m.get("mask")
    out = attend(scores, vh, causal(pos, n, mask["size"] if mask else None))
    out = out * torch.sigmoid(h @ _w(p["g"]).T)
    return out @ _w(p["o"]).T + _w(p["o.b"])


def attention_2_cache(h, p, m, pos0, eps):
    T = h.shape[0]
    k = norm_plain(h @ _w(p["k"]).T, p["k.norm"], eps).view(T, m["kv_heads"], m["dim"])
    k = rotate_half(k, torch.arange(pos0, pos0 + T), frequencies_by_wavelength(m["rot"]))
    v = (h @ _w(p["v"]).T).view(T, m["kv_heads"], m["vdim"])
    return k, v


def attention_2(h, p, m, pos0, cache, eps, sink=True):
    T, H, G, D, V = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    keys, values = cache
    n = keys.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    q = norm_plain(h @ _w(p["q"]).T, p["q.norm"], eps).view(T, H, D)
    q = rotate_half(q, pos, frequencies_by_wavelength(m["rot"]))
    rep = H // G
    kh = keys.repeat_interleave(rep, dim=1).permute(1, 0, 2)
    vh = values.repeat_interleave(rep, dim=1).permute(1, 0, 2)
    scores = torch.einsum("thd,hnd->htn", q, kh) * float(m["scale"])
    cap = float(m["softcap"])
    scores = cap * torch.tanh(scores / cap)
    out = attend(scores, vh, causal(pos, n), _w(p["sink"]) if sink else None)
    gate = torch.sigmoid(h @ _w(p["g"]).T)                              # [T, H]
    out = (out.view(T, H, V) * gate.unsqueeze(-1)).reshape(T, H * V)
    return out @ _w(p["o"]).T


def latent_cache(h, p, m, pos0, eps):
    """The latent and the rotated key part of the tokens h: all that a ``latent_attention`` layer caches."""
    T, R = h.shape[0], m["kv_rank"]
    d = h @ _w(p["dkv"]).T
    c = norm_plain(d[:, :R], p["dkv.norm"], eps)
    freqs, mag = frequencies_ramped(m["rot"])
    r = rotate_pairs(d[:, R:].view(T, 1, -1), torch.arange(pos0, pos0 + T), freqs, mag).view(T, -1)
    return c, r


def latent_attention(h, p, m, pos0, cache, eps, sink=True):
    T, H, D, Rd, V = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, r = cache
    n = c.shape[0]
    pos = torch.arange(pos0, pos0 + T)
    cq = norm_plain(h @ _w(p["dq"]).T, p["dq.norm"], eps)
    q = (cq @ _w(p["uq"]).T).view(T, H, D + Rd)
    freqs, mag = frequencies_ramped(m["rot"])
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], pos, freqs, mag)
    k_plain = (c @ _w(p["uk"]).T).view(n, H, D)
    v = (c @ _w(p["uv"]).T).view(n, H, V)
    scores = (torch.einsum("thd,nhd->htn", q_plain, k_plain) + torch.einsum("thd,nd->htn", q_rot, r)) * float(m["scale"])
    mask = m.get("mask")
    out = attend(scores, v.permute(1, 0, 2), causal(pos, n, mask["size"] if mask else None), _w(p["sink"]) if sink else None)
    return out @ _w(p["o"]).T


# --------------------------------------------------------------------------------------- feed-forward
def expert(h, gate, up, down, limit):
    g = torch.clamp(h @ _w(gate).T, max=limit)
    u = torch.clamp(h @ _w(up).T, min=-limit, max=limit)
    return (g * torch.sigmoid(ACT_ALPHA * g) * (u + 1.0)) @ _w(down).T


def route(z, top):
    """(experts, weights) for one token's router logits: the ``top`` largest (the earlier wins a tie), softmax over them."""
    order = sorted(range(z.numel()), key=lambda e: (-float(z[e]), e))[:top]
    w = torch.softmax(z[order], dim=0)
    return order, w


def feed_forward(h, p, mlp):
    if mlp is None:
        return torch.zeros_like(h)
    z = h @ _w(p["router"]).T + _w(p["router.b"])
    out = torch.zeros_like(h)
    lim = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        chosen, w = route(z[t], mlp["router"]["top"])
        for e, we in zip(chosen, w):
            out[t] += we * expert(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"], lim)[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, p["shared.gate"], p["shared.up"], p["shared.down"], float(mlp["shared"]["limit"]))
    return out


# ---------------------------------------------------------------------------------------------- model
def _sub(w, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in w.items() if k.startswith(prefix)}


class Plain:
    """The whole model with a cache per layer run, so that a prompt can be fed in portions."""

    def __init__(self, cfg, weights, sink=True):
        self.cfg, self.w, self.sink = cfg, weights, sink
        self.eps = float(cfg["norm"]["eps"])
        self.runs = layer_runs(cfg)
        self.cache = [None] * len(self.runs)
        self.pos = 0

    def _mixer(self, r, layer, h):
        spec = self.cfg["layers"][layer]
        m, kind = spec["mixer"], spec["type"]
        p = _sub(self.w, f"l{layer}.mix.")
        if kind == "attention":
            new = attention_cache(h, p, m, self.pos)
        elif kind == "attention_2":
            new = attention_2_cache(h, p, m, self.pos, self.eps)
        elif kind == "latent_attention":
            new = latent_cache(h, p, m, self.pos, self.eps)
        else:
            raise ValueError(kind)
        old = self.cache[r]
        self.cache[r] = new if old is None else tuple(torch.cat([a, b]) for a, b in zip(old, new))
        if kind == "attention":
            return attention(h, p, m, self.pos, self.cache[r])
        if kind == "attention_2":
            return attention_2(h, p, m, self.pos, self.cache[r], self.eps, self.sink)
        return latent_attention(h, p, m, self.pos, self.cache[r], self.eps, self.sink)

    def forward(self, tokens, streams=None):
        """Logits [T, vocab] of the next portion ``tokens``; ``streams`` (a list) receives the stream after every layer run."""
        x0 = _w(self.w["embed"][torch.tensor(tokens)])
        x = x0.clone()
        for r, (layer, _, first) in enumerate(self.runs):
            if first:
                x = x + x0
            h = norm_one_plus(x, self.w[f"l{layer}.norm1"], self.eps)
            x = x + (self._mixer(r, layer, h) + feed_forward(h, _sub(self.w, f"l{layer}.mlp."), self.cfg["layers"][layer].get("mlp")))
            if streams is not None:
                streams.append(x.clone())
        self.pos += len(tokens)
        return norm_one_plus(x, self.w["final.norm"], self.eps) @ _w(self.w["head"]).T
