"""A plain, slow implementation of the Vumezen design in 64-bit arithmetic: the oracle of the tests.

One function per mechanism, written from the design's equations; it shares no code with the engine.
Weights come as a dictionary name -> tensor (any floating type; widened to float64), the configuration as
the dictionary of config.json.

The design in short.  Embedding: table row times a scale, plus a row of a second table chosen by a hash of
(previous token, token); a sequence's first token takes that table's last row.  A layer adds BOTH
sublayers' outputs to the stream they both read: x <- x + mixer(norm1(x)) + ff(norm2(x)).  The mixer is
grouped-query attention without biases: rotation of the first ``rot.dims`` dimensions of each query and key
head (pairs (i, i + dims/2)), an explicit score scale, a causal sliding window that also keeps the
sequence's first tokens visible, a softmax whose denominator counts one more (a sink without a value),
values of their own size.  A layer may take its keys and values from an earlier layer's cache.  The
feed-forward is a mixture of relu-squared experts chosen by sigmoid scores plus a correction, weighted by the
uncorrected scores times a scale, beside a shared expert.
"""
from __future__ import annotations

import torch

F64 = torch.float64
SINK = 1.0          # what the softmax's denominator counts beside the keys (a test sets 0 to show that it matters)


def _w(t):
    return t.to(F64)


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * _w(weight)


# ----------------------------------------------------------------------------------- embedding
def bigram_row(prev, token, e):
    """Row of the second table: the hash of the pair, or the last row for a sequence's first token."""
    b = e["bigram"]
    if prev is None:
        return b["buckets"]
    return (prev * b["mul_prev"] + token * b["mul_cur"]) % b["buckets"]


def embed(tokens, prev, w, e):
    """``prev``: the token before ``tokens[0]`` (None at a sequence's start).  [T, W]."""
    rows = []
    for t in tokens:
        x = _w(w["embed"][t]) * float(e["scale"])
        if e.get("bigram") is not None:
            x = x + _w(w["bigram"][bigram_row(prev, t, e)])
        rows.append(x)
        prev = t
    return torch.stack(rows)


# ----------------------------------------------------------------------------------- attention
def rotate(x, positions, dims, base):
    """x [T, heads, d]: the first ``dims`` dimensions in pairs (i, i + dims/2); angle position * base^(-2i/dims)."""
    if not dims:
        return x
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = positions.to(F64).unsqueeze(-1) * f
    c, s = torch.cos(a).unsqueeze(1), torch.sin(a).unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def _rot(m):
    """(dims, base) of a mixer's rotation; a mixer whose configuration names none does not rotate."""
    rot = m.get("rot")
    return (0, 1.0) if rot is None else (int(rot["dims"]), float(rot["base"]))


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def project_kv(h, p, m, pos0):
    """Keys (rotated) and values of the tokens ``h`` at positions pos0..: what a layer's cache holds."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    pos = torch.arange(pos0, pos0 + T)
    k = rotate((h @ _w(p["k"]).T).view(T, G, D), pos, *_rot(m))
    v = (h @ _w(p["v"]).T).view(T, G, V)
    return k, v


def attend(h, p, m, pos0, keys, values):
    """The mixer's output for the tokens ``h`` (positions pos0..) over ``keys``/``values`` [n, G, .], which
    hold every position from 0 up to the last of these tokens."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
    mask = m.get("mask") or {"size": 1 << 60}          # no mask named: plain causal attention
    size, keep = mask["size"], mask.get("keep_first", 0)
    pos = torch.arange(pos0, pos0 + T)
    q = rotate((h @ _w(p["q"]).T).view(T, H, D), pos, *_rot(m))
    out = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        i = pos0 + t
        js = torch.tensor([j for j in range(i + 1) if visible(i, j, size, keep)])
        ks, vs = keys[js], values[js]
        for hd in range(H):
            g = hd // (H // G)
            s = (ks[:, g] @ q[t, hd]) * float(m["scale"])
            mx = torch.clamp(s.max(), min=0.0)
            ex = torch.exp(s - mx)
            pr = ex / (SINK * torch.exp(-mx) + ex.sum())
            out[t, hd] = pr @ vs[:, g]
    return out.reshape(T, H * V) @ _w(p["o"]).T


# -------------------------------------------------------------------------------- feed-forward
def relu2_expert(h, up, down):
    return torch.relu(h @ _w(up).T).pow(2) @ _w(down).T


def choose(scores, correction, top):
    """Indices of the ``top`` largest of scores + correction (the earlier index wins a tie)."""
    c = scores + correction
    order = sorted(range(c.numel()), key=lambda e: (-float(c[e]), e))
    return order[:top]


def moe(h, p, mlp):
    r = mlp["router"]
    E, top, scale = r["experts"], r["top"], float(r.get("scale", 1.0))
    out = torch.zeros_like(h)
    s = torch.sigmoid(h @ _w(p["router"]).T)
    corr = _w(p["correction"]) if "correction" in p else torch.zeros(E, dtype=F64)
    for t in range(h.shape[0]):
        for e in choose(s[t], corr, top):
            out[t] += scale * s[t, e] * relu2_expert(h[t:t + 1], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + relu2_expert(h, p["shared.up"], p["shared.down"])
    return out


# --------------------------------------------------------------------------------------- model
def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


class PlainVumezen:
    """Keeps a sequence's keys, values and last token, so that it can be fed in pieces."""

    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights
        self.pos, self.prev = 0, None
        self.kv = [None] * len(cfg["layers"])
        self.trace = []        # the residual stream after every layer of the last call

    def forward(self, tokens):
        cfg, w = self.cfg, self.w
        eps = float(cfg["norm"]["eps"])
        x = embed(tokens, self.prev, w, cfg["embedding"])
        self.trace = []
        for i, lay in enumerate(cfg["layers"]):
            m = lay["mixer"]
            a = rms_norm(x, w[f"l{i}.norm1"], eps)
            p = sub(w, f"l{i}.mix.")
            src = m.get("kv_from")
            if src is None:
                k, v = project_kv(a, p, m, self.pos)
                old = self.kv[i]
                self.kv[i] = (k, v) if old is None else (torch.cat([old[0], k]), torch.cat([old[1], v]))
                src = i
            update = attend(a, p, m, self.pos, *self.kv[src])
            if lay.get("mlp") is not None:
                update = update + moe(rms_norm(x, w[f"l{i}.norm2"], eps), sub(w, f"l{i}.mlp."), lay["mlp"])
            x = x + update
            self.trace.append(x.clone())
        self.pos += len(tokens)
        self.prev = tokens[-1]
        return rms_norm(x, w["final.norm"], eps) @ _w(w["head"]).T
