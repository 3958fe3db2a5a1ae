"""Small Vumezen configurations and weights for the tests, made here from seeds.

The configurations differ from one another in every size and option: heads and groups of heads, key sizes
and value sizes (larger, smaller, equal), rotations of part of a head, of the whole head and none, windows
with several, one and no kept first tokens, layers that read another layer's keys and values with a mask
of their own, routers with and without a scale, one expert chosen and several, layers without a shared
expert or without a feed-forward, embeddings with and without the table of token pairs.
"""
from __future__ import annotations

import copy
import json
import os
import random

import torch

import plain_vumezen as P


def att(heads, kv_heads, dim, vdim, scale, window, keep, rot_dims=None, base=10000.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": window, "keep_first": keep}}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def moe(ff, experts, top, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": "attention", "mixer": copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)}


def config(vocab, width, layers, eps=1e-5, scale=4.0, bigram=(53, 31, 7)):
    emb = {"scale": scale}
    if bigram is not None:
        emb["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return {"architecture": "Vumezen", "vocab": vocab, "width": width, "embedding": emb, "layers": layers, "norm": {"eps": eps}}


# attention scores are made peaky (scale well above 1/sqrt(size)) so that a key that is lost, one too many or one too
# few at a window's edge, or a kept first token that is dropped changes the result by much more than any tolerance
A = att(4, 2, 16, 24, 0.7, 12, 3, rot_dims=8, base=1000.0)
B = att(1, 1, 32, 16, 0.5, 9, 0, rot_dims=32, base=300.0)
C = att(3, 1, 10, 6, 0.9, 7, 1, rot_dims=6, base=50.0)
CONFIGS = {
    # every mechanism: groups of two query heads, values larger than keys, a reader whose window and kept tokens differ
    # from its writer's (larger and smaller), a layer without a feed-forward
    "mix": config(211, 64, [
        layer(A, moe(24, 6, 2, scale=1.5, shared=40)),
        layer({**A, "mask": {"size": 20, "keep_first": 1}, "scale": 0.5, "kv_from": 0}, moe(24, 6, 2, scale=1.5, shared=40)),
        layer(A, None),
        layer({**A, "mask": {"size": 5, "keep_first": 6}, "kv_from": 2}, moe(16, 4, 3, shared=8)),
    ]),
    # one head; the whole head rotates; values smaller than keys; no kept tokens; one expert chosen, no scale, no shared
    # expert; no table of token pairs; a reader two layers after its writer
    "alt": config(157, 96, [
        layer(B, moe(56, 4, 1)),
        layer(att(2, 2, 8, 8, 1.2, 30, 2), None),                       # no rotation at all; its window is never left
        layer({**B, "mask": {"size": 4, "keep_first": 0}, "kv_from": 0}, moe(56, 5, 2, scale=0.5, shared=24)),
    ], eps=3e-6, scale=1.0, bigram=None),
    # sizes that are multiples of nothing: every product falls to the CUDA-core kernels
    "odd": config(97, 44, [
        layer(C, moe(18, 3, 2, scale=2.5, shared=10)),
        layer({**C, "kv_from": 0}, moe(18, 3, 3)),
    ], scale=2.0, bigram=(17, 5, 11)),
}
MECHANISMS = {
    "attention_alone": config(61, 32, [layer(att(2, 1, 8, 8, 1.2, 1000, 0, rot_dims=8), None)], scale=1.0, bigram=None),
    "window_and_kept_tokens": config(61, 32, [layer(att(2, 1, 8, 8, 1.2, 6, 2, rot_dims=4), None)], scale=1.0, bigram=None),
    "window_of_one": config(61, 32, [layer(att(2, 2, 8, 8, 1.2, 1, 1, rot_dims=4), None)], scale=1.0, bigram=None),
    "values_of_their_own_size": config(61, 32, [layer(att(2, 1, 8, 20, 1.2, 9, 1, rot_dims=8), None)], scale=1.0, bigram=None),
    "values_wider_than_a_warp": config(61, 32, [layer(att(2, 1, 8, 72, 1.2, 9, 1, rot_dims=8), None)], scale=1.0, bigram=None),
    "another_layers_keys": config(61, 32, [layer(att(2, 1, 8, 12, 1.2, 7, 2, rot_dims=4), None),
                                           layer(att(2, 1, 8, 12, 0.6, 11, 0, rot_dims=4, kv_from=0), None)], scale=1.0, bigram=None),
    "token_pairs": config(61, 32, [layer(att(2, 1, 8, 8, 0.1, 5, 0), None)], scale=3.0, bigram=(7, 3, 5)),
    "experts": config(61, 32, [layer(att(2, 1, 8, 8, 0.3, 8, 1, rot_dims=8), moe(20, 8, 3, scale=2.5, shared=12))], bigram=None),
    "experts_one_of_two": config(61, 32, [layer(att(2, 1, 8, 8, 0.3, 8, 1, rot_dims=8), moe(20, 2, 1))], bigram=None),
}


def tensor_shapes(cfg):
    """Names and shapes of a configuration's tensors, from the design's naming (no engine code)."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    if cfg["embedding"].get("bigram"):
        out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
        out.update({p + "norm1": (W,), p + "mix.q": (H * D, W), p + "mix.o": (W, H * V)})
        if m.get("kv_from") is None:
            out.update({p + "mix.k": (G * D, W), p + "mix.v": (G * V, W)})
        mlp = lay["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (W,)
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            out.update({f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
        out.update({p + "mlp.router": (mlp["router"]["experts"], W), p + "mlp.correction": (mlp["router"]["experts"],)})
        if mlp.get("shared"):
            out.update({p + "mlp.shared.up": (mlp["shared"]["ff"], W), p + "mlp.shared.down": (W, mlp["shared"]["ff"])})
    return out


def make_weights(cfg, seed):
    """bfloat16-representable weights: matrices with unit-sized outputs, norms near 1, router matrices large (clear
    choices) with a correction that changes choices, a pair table as large as the embedding."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        r = lambda: torch.randn(shape, generator=gen)
        if name.endswith(("norm", "norm1", "norm2")):
            t = 1.0 + 0.2 * (torch.rand(shape, generator=gen) - 0.5)
        elif name.endswith("router"):
            t = 6.0 * r() / shape[-1] ** 0.5
        elif name.endswith("correction"):
            t = 0.3 * r()
        elif name == "embed":
            t = r()
        elif name == "bigram":
            t = float(cfg["embedding"]["scale"]) * r()
        else:
            t = r() / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(path, cfg, weights):
    from zinfer_b200.weights import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in weights.items()})
    return path


def plain_logits(cfg, weights, reqs):
    return {rid: P.PlainVumezen(cfg, weights).forward(toks).numpy() for rid, toks in reqs.items()}


def clear_requests(cfg, weights, lengths, seed, margin):
    """Requests whose every choice of experts is clear by ``margin`` in the plain model (a choice that bfloat16 cannot
    tell apart would be no fault of the engine's).  Built token by token: the plain model keeps its keys, values and
    last token, a candidate token is fed, and if one of its choices is unclear everything is put back and another is tried."""
    rng = random.Random(seed)
    has_moe = any(lay["mlp"] for lay in cfg["layers"])
    margins = []
    orig = P.choose

    def spy(scores, correction, top):
        c = (scores + correction).sort(descending=True).values
        margins.append(float(c[top - 1] - c[top]) if top < c.numel() else float("inf"))
        return orig(scores, correction, top)

    reqs = {}
    P.choose = spy
    try:
        for r, n in enumerate(lengths):
            model, toks = P.PlainVumezen(cfg, weights), []
            while len(toks) < n:
                for _ in range(300):
                    cand = rng.randrange(cfg["vocab"])
                    if not has_moe:
                        break
                    saved = (list(model.kv), model.pos, model.prev)
                    del margins[:]
                    model.forward([cand])
                    if min(margins) >= margin:
                        break
                    model.kv, model.pos, model.prev = saved
                else:
                    raise AssertionError("no candidate token with clear choices of experts")
                toks.append(cand)
            reqs[f"r{r}"] = toks
    finally:
        P.choose = orig
    return reqs
