"""Small Sepitar configurations and weights for the tests, made here from seeds.

The configurations differ from one another in every size and option: heads and groups of heads, key sizes and
value sizes (larger, smaller, equal), rotations of part of a head and of the whole head, windows and none, distance
tables of several sizes, latent ranks, experts chosen one and several, layers without a shared expert or without a
feed-forward, ranges of layers run once, twice and three times, from the first layer and from a later one.
"""
from __future__ import annotations

import copy
import json
import os
import random

import torch

import plain_sepitar as P


def att(heads, kv_heads, dim, vdim, scale, window, bias_max):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max}
    if window:
        m["mask"] = {"size": window}
    return m


def att2(heads, kv_heads, dim, vdim, scale, softcap, rot_dims, base=1000.0, scaling=(4.0, 1.0, 4.0, 64)):
    factor, low, high, original = scaling
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
            "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor, "low": low, "high": high, "original": original}}}


def lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, window, base=500.0, scaling=(4.0, 32, 8.0, 1.0)):
    factor, original, fast, slow = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}}
    if window:
        m["mask"] = {"size": window}
    return m


def moe(ff, experts, top, limit, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)}


def config(vocab, width, layers, loop=None, eps=1e-5, rel_rows=None):
    """``rel_rows``: rows of the distance tables per layer index (the tensors' shape gives them, not config.json)."""
    cfg = {"architecture": "Sepitar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    cfg["_rel_rows"] = rel_rows or {}
    return cfg


def public(cfg):
    """The configuration as config.json has it (without the tests' own notes)."""
    return {k: v for k, v in cfg.items() if not k.startswith("_")}


# attention scores are made peaky (scales well above 1/sqrt(size)) so that a key that is lost, or one too many or too
# few at a window's edge, changes the result by much more than any tolerance
A = att(4, 2, 16, 24, 0.6, 9, 40)
A2 = att2(4, 2, 16, 8, 0.5, 5.0, 8)
L = lat(3, 8, 4, 12, 20, 10, 0.5, 11)
CONFIGS = {
    # every mechanism: three passes over layers 1..2; values larger and smaller than keys; groups of two query heads;
    # a layer without a feed-forward; one without a shared expert
    "mix": config(211, 64, [
        layer("latent_attention", L, moe(24, 6, 2, 1.5, shared=(40, 2.0))),
        layer("attention", A, moe(24, 6, 2, 1.5)),
        layer("attention_2", A2, None),
        layer("latent_attention", {**L, "mask": {"size": 5}}, moe(16, 4, 3, 0.8, shared=(8, 1.0))),
    ], loop=(1, 3, 3), rel_rows={1: 12}),
    # no loop; attention without a window; one head per group; the whole head rotates; one expert chosen; latent
    # attention without a window
    "alt": config(157, 96, [
        layer("attention_2", att2(2, 2, 32, 32, 0.3, 30.0, 32, base=300.0, scaling=(8.0, 1.0, 2.0, 16)), moe(56, 4, 1, 3.0)),
        layer("attention", att(1, 1, 32, 16, 0.4, 0, 25), moe(56, 5, 2, 1.0, shared=(24, 0.5))),
        layer("latent_attention", lat(2, 16, 8, 16, 32, 24, 0.35, 0, base=100.0, scaling=(2.0, 16, 4.0, 2.0)), None),
    ], eps=3e-6, rel_rows={1: 8}),
    # sizes that are multiples of nothing: every product falls to the CUDA-core kernels; the loop starts at layer 0 and
    # covers everything
    "odd": config(97, 44, [
        layer("attention", att(3, 1, 10, 6, 0.7, 7, 13), moe(18, 3, 2, 2.5, shared=(10, 1.2))),
        layer("latent_attention", lat(3, 6, 6, 10, 14, 9, 0.6, 13, base=50.0), moe(18, 3, 3, 0.6)),
        layer("attention_2", att2(3, 1, 10, 14, 0.8, 2.0, 6, base=50.0), moe(10, 2, 1, 1.0, shared=(6, 3.0))),
    ], loop=(0, 3, 2), rel_rows={0: 6}),
}
MECHANISMS = {
    "attention_alone": config(61, 32, [layer("attention", att(2, 1, 8, 8, 0.9, 6, 20), None)], rel_rows={0: 10}),
    "attention_without_a_window": config(61, 32, [layer("attention", att(2, 2, 8, 12, 0.9, 0, 30), None)], rel_rows={0: 16}),
    "attention_window_of_one": config(61, 32, [layer("attention", att(2, 1, 8, 8, 0.9, 1, 9), None)], rel_rows={0: 4}),
    "attention_2_alone": config(61, 32, [layer("attention_2", att2(2, 1, 8, 8, 0.9, 3.0, 4), None)]),
    "attention_2_wide_values": config(61, 32, [layer("attention_2", att2(2, 1, 8, 72, 0.9, 50.0, 8), None)]),
    "latent_alone": config(61, 32, [layer("latent_attention", lat(2, 8, 4, 8, 12, 6, 0.7, 6), None)]),
    "latent_without_a_window": config(61, 32, [layer("latent_attention", lat(2, 8, 8, 6, 16, 8, 0.7, 0), None)]),
    "experts": config(61, 32, [layer("attention_2", att2(2, 1, 8, 8, 0.3, 10.0, 8), moe(20, 8, 3, 1.0, shared=(12, 0.7)))]),
    "experts_one_of_two": config(61, 32, [layer("attention_2", att2(2, 1, 8, 8, 0.3, 10.0, 8), moe(20, 2, 1, 2.0))]),
    "layers_run_three_times": config(61, 32, [layer("latent_attention", lat(2, 8, 4, 8, 12, 6, 0.7, 6), None),
                                              layer("attention", att(2, 1, 8, 8, 0.9, 5, 12), None)], loop=(1, 2, 3),
                                     rel_rows={1: 6}),
}


def tensor_shapes(cfg):
    """Names and shapes of a configuration's tensors, from the design's naming (no engine code)."""
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    for i, lay in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", lay["mixer"], lay["type"]
        out[p + "norm1"] = (W,)
        H = m["heads"]
        if kind == "latent_attention":
            D, R, V = m["dim"], m["rot_dim"], m["vdim"]
            out.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * (D + R), m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"] + R, W), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * D, m["kv_rank"]),
                        p + "mix.uv": (H * V, m["kv_rank"]), p + "mix.sink": (H,), p + "mix.o": (W, H * V)})
        else:
            G, D, V = m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, W), p + "mix.k": (G * D, W), p + "mix.v": (G * V, W), p + "mix.o": (W, H * V)})
            if kind == "attention":
                out.update({p + "mix.q.b": (H * D,), p + "mix.k.b": (G * D,), p + "mix.v.b": (G * V,), p + "mix.o.b": (W,),
                            p + "mix.rel": (cfg["_rel_rows"][i], H), p + "mix.g": (H * V, W)})
            else:
                out.update({p + "mix.q.norm": (H * D,), p + "mix.k.norm": (G * D,), p + "mix.sink": (H,), p + "mix.g": (H, W)})
        mlp = lay["mlp"]
        if mlp is None:
            continue
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            out.update({f"{p}mlp.e{e}.gate": (ff, W), f"{p}mlp.e{e}.up": (ff, W), f"{p}mlp.e{e}.down": (W, ff)})
        out.update({p + "mlp.router": (mlp["router"]["experts"], W), p + "mlp.router.b": (mlp["router"]["experts"],)})
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    return out


def make_weights(cfg, seed):
    """bfloat16-representable weights: matrices with unit-sized outputs, norm weights around zero (the design adds
    one), router matrices large (clear choices) with a bias that changes choices, sinks and distance tables as large
    as the scores, gate and up matrices large enough that the experts' clamps bite."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        r = lambda: torch.randn(shape, generator=gen)
        if name.endswith(("norm1", "final.norm")):
            t = 0.4 * (torch.rand(shape, generator=gen) - 0.5)
        elif name.endswith(".norm"):
            t = 1.0 + 0.4 * (torch.rand(shape, generator=gen) - 0.5)
        elif name.endswith("router"):
            t = 6.0 * r() / shape[-1] ** 0.5
        elif name.endswith("router.b"):
            t = 1.5 * r()
        elif name.endswith((".sink", ".rel")):
            t = 1.5 * r()
        elif name.endswith(".b"):
            t = 0.5 * r()
        elif name == "embed":
            t = r()
        elif name.endswith((".gate", ".up")):
            t = 2.0 * r() / shape[-1] ** 0.5
        else:
            t = r() / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(path, cfg, weights):
    from zinfer_b200.weights import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(public(cfg), f)
    write_safetensors(os.path.join(path, "model.safetensors"), {k: v.contiguous() for k, v in weights.items()})
    return path


def plain_logits(cfg, weights, reqs, **kw):
    return {rid: P.Plain(cfg, weights, **kw).forward(toks).numpy() for rid, toks in reqs.items()}


def clear_requests(cfg, weights, lengths, seed, margin):
    """Requests whose every choice of experts is clear by ``margin`` in the plain model (a choice that bfloat16 cannot
    tell apart would be no fault of the engine's).  Built token by token: the plain model keeps its caches, a candidate
    token is fed, and if one of its choices is unclear everything is put back and another is tried."""
    rng = random.Random(seed)
    has_moe = any(lay["mlp"] for lay in cfg["layers"])
    margins = []
    orig = P.route

    def spy(z, top):
        c = z.sort(descending=True).values
        margins.append(float(c[top - 1] - c[top]) if top < c.numel() else float("inf"))
        return orig(z, top)

    reqs = {}
    P.route = spy
    try:
        for r, n in enumerate(lengths):
            if not has_moe:
                reqs[f"r{r}"] = [rng.randrange(cfg["vocab"]) for _ in range(n)]
                continue
            model, toks = P.Plain(cfg, weights), []
            while len(toks) < n:
                for _ in range(300):
                    cand = rng.randrange(cfg["vocab"])
                    saved = (list(model.cache), model.pos)
                    del margins[:]
                    model.forward([cand])
                    if min(margins) >= margin:
                        break
                    model.cache, model.pos = saved
                else:
                    raise AssertionError("no candidate token with clear choices of experts")
                toks.append(cand)
            reqs[f"r{r}"] = toks
    finally:
        P.route = orig
    return reqs
