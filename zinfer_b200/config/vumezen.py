"""Typed configuration of the Vumezen design and its model spec.

A Vumezen model is a decoder whose layers add BOTH sublayers' outputs to the stream they both read,
x <- x + mixer(norm1(x)) + ff(norm2(x)).  The embedding is a table row times ``embedding.scale`` plus a row of a
second table chosen by a hash of the token and the one before it.  The mixer is grouped-query attention without
biases or head norms: the first ``rot.dims`` dimensions of each query and key head rotate, the score has an explicit
``scale``, the mask is causal within ``mask.size`` tokens and also keeps a sequence's first ``mask.keep_first`` tokens
visible, the softmax's denominator counts one more than the keys (a sink), and values have a size of their own
(``vdim``).  A mixer with ``kv_from: j`` has no key and value projections: it reads the cache of layer ``j``.  The
feed-forward is a mixture of relu-squared experts (sigmoid scores, a correction added for the choice only, weights =
scores times ``router.scale``, no renormalisation) beside a shared expert, or absent.  config.json gives every size
and every constant that may differ between models; the tensor names (``embed``, ``bigram``, ``l<i>.norm1``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``) are fixed.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Optional

from .luvavik import _positive
from .qwen3 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Vumezen"
DEFAULT_MAX_POSITIONS = 1 << 17       # the design has no position limit; the engine needs one for its tables
SINK = 1.0                            # what the softmax's denominator counts beside the keys: fixed by the design

_MIXER_KEYS = ("heads", "kv_heads", "dim", "scale")


@dataclass(frozen=True)
class VumezenConfig:
    vocab_size: int
    hidden_size: int
    layers: tuple[dict, ...]               # as in config.json: type, mixer, mlp
    norm_eps: float
    embedding: dict                        # scale, and bigram: buckets, mul_prev, mul_cur (or no bigram)
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)
    model_type: str = "vumezen"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "VumezenConfig":
        for k in ("vocab", "width", "layers", "norm"):
            if k not in d:
                raise ConfigError(f"config.json lacks required key {k!r}")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("config.json: `layers` must be a list with at least one layer")
        if "eps" not in d["norm"]:
            raise ConfigError("config.json: norm lacks 'eps'")
        eos = d.get("eos_token_id", ())
        if isinstance(eos, int):
            eos = (eos,)
        cfg = cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                  layers=tuple(copy.deepcopy(layer) for layer in d["layers"]), norm_eps=float(d["norm"]["eps"]),
                  embedding=copy.deepcopy(d.get("embedding") or {}),
                  max_position_embeddings=int(d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=tuple(int(t) for t in (eos or ())))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps >= 0.0:
            raise ConfigError(f"norm.eps must be >= 0, got {self.norm_eps}")
        bigram = self.embedding.get("bigram")
        if bigram is not None:
            for k in ("buckets", "mul_prev", "mul_cur"):
                if k not in bigram:
                    raise ConfigError(f"config.json: embedding.bigram lacks {k!r}")
            if int(bigram["buckets"]) <= 0:
                raise ConfigError("config.json: embedding.bigram wants at least one bucket")
        for i, layer in enumerate(self.layers):
            kind, m = layer.get("type"), layer.get("mixer")
            if kind != "attention":
                raise ConfigError(f"config.json: layer {i} has the unknown mixer type {kind!r}; known: attention")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: layer {i} lacks its mixer's sizes")
            where = f"layers[{i}].mixer"
            _positive(where, m, _MIXER_KEYS)
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {where}: {m['heads']} heads do not divide into {m['kv_heads']} kv heads")
            if int(m.get("vdim", m["dim"])) <= 0:
                raise ConfigError(f"config.json: {where}.vdim must be positive")
            rot = m.get("rot")
            if rot is not None:
                _positive(f"{where}.rot", rot, ("base", "dims"))
                if rot["dims"] % 2 or rot["dims"] > m["dim"]:
                    raise ConfigError(f"config.json: {where}.rot.dims {rot['dims']} must be even and at most dim")
            mask = m.get("mask")
            if mask is not None:
                _positive(f"{where}.mask", mask, ("size",))
                if int(mask.get("keep_first", 0)) < 0:
                    raise ConfigError(f"config.json: {where}.mask.keep_first must not be negative")
            src = m.get("kv_from")
            if src is not None:
                if not isinstance(src, int) or not 0 <= src < i:
                    raise ConfigError(f"config.json: {where}.kv_from {src!r} must name an earlier layer")
                other = self.layers[src]["mixer"]
                if other.get("kv_from") is not None:
                    raise ConfigError(f"config.json: {where}.kv_from names layer {src}, which has no keys and values of its own")
                same = ("kv_heads", "dim", "heads")
                if any(other.get(k) != m.get(k) for k in same) or int(other.get("vdim", other["dim"])) != int(m.get("vdim", m["dim"])) \
                        or (other.get("rot") or {}) != (m.get("rot") or {}):
                    raise ConfigError(f"config.json: {where}.kv_from: layer {src}'s heads, sizes and rotation differ from this layer's")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind", "moe") != "moe":
                raise ConfigError(f"config.json: layer {i} has the unknown feed-forward kind {mlp.get('kind')!r}; known: moe")
            _positive(f"layers[{i}].mlp.expert", mlp.get("expert") or {}, ("ff",))
            router = mlp.get("router") or {}
            _positive(f"layers[{i}].mlp.router", router, ("experts", "top"))
            if router["top"] > router["experts"]:
                raise ConfigError(f"config.json: layer {i}: {router['top']} of {router['experts']} experts cannot be chosen")
            if mlp.get("shared") is not None:
                _positive(f"layers[{i}].mlp.shared", mlp["shared"], ("ff",))

    def describe(self) -> list[str]:
        """Lines for the command line's model inspection."""
        e = self.embedding
        b = e.get("bigram")
        lines = [f"hidden_size: {self.hidden_size}", f"vocab_size: {self.vocab_size}", f"num_layers: {len(self.layers)}",
                 f"norm_eps: {self.norm_eps:e}",
                 f"embedding: scale {float(e.get('scale', 1.0))}" + (
                     f", token pairs in {b['buckets']} buckets (previous x {b['mul_prev']} + token x {b['mul_cur']})" if b else "")]
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            mask, rot = m.get("mask"), m.get("rot")
            mixer = (f"heads={m['heads']} kv_heads={m['kv_heads']} dim={m['dim']} vdim={m.get('vdim', m['dim'])} scale={m['scale']}"
                     + (f" rot dims={rot['dims']} base={rot['base']}" if rot else " no rotation")
                     + (f" window={mask['size']} keep_first={mask.get('keep_first', 0)}" if mask else " no window")
                     + (f" keys and values of layer {m['kv_from']}" if m.get("kv_from") is not None else ""))
            mlp = layer.get("mlp")
            if mlp is None:
                ff = "none"
            else:
                r = mlp["router"]
                ff = (f"moe experts={r['experts']} top={r['top']} scale={r.get('scale', 1.0)} ff={mlp['expert']['ff']}"
                      + (f" shared ff={mlp['shared']['ff']}" if mlp.get("shared") else ""))
            lines.append(f"layer {i}: attention ({mixer}); feed-forward: {ff}")
        return lines

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "embedding": copy.deepcopy(self.embedding),
                             "layers": [copy.deepcopy(layer) for layer in self.layers], "norm": {"eps": self.norm_eps}}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d


# ---------------------------------------------------------------------- the family
def _mixer_spec(cfg: VumezenConfig, m: dict) -> PartSpec:
    rot, mask = m.get("rot"), m.get("mask")
    position = None
    if rot is not None:
        position = PartSpec("rope", {"head_dim": int(rot["dims"]), "theta": float(rot["base"]),
                                     "max_positions": cfg.max_position_embeddings})
    return PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
        "head_dim": int(m["dim"]), "value_dim": int(m.get("vdim", m["dim"])), "qk_norm_eps": None,
        "window": int(mask["size"]) if mask else None, "keep_first": int(mask.get("keep_first", 0)) if mask else 0,
        "position": position, "scale": float(m["scale"]), "sink": SINK, "projects_kv": m.get("kv_from") is None,
        "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})


def _ffn_spec(cfg: VumezenConfig, layer: dict) -> Optional[PartSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    H = cfg.hidden_size
    router = mlp["router"]
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("plain_mlp", {"hidden_size": H, "intermediate_size": int(mlp["shared"]["ff"]), "activation": "relu2",
                                        "names": ("up", "down")})
    return PartSpec("routed_experts", {
        "hidden_size": H, "intermediate_size": int(mlp["expert"]["ff"]), "experts": int(router["experts"]),
        "top": int(router["top"]), "renormalize": False, "correction": True, "activation": "relu2", "score": "sigmoid",
        "weight_scale": float(router.get("scale", 1.0)), "expert_names": "e{}.", "shared": shared, "shared_name": "shared."})


def vumezen_model_spec(cfg: VumezenConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = lambda tensor: PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": tensor})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        ffn = _ffn_spec(cfg, layer)
        block = PartSpec("parallel_block", {
            "mixer": _mixer_spec(cfg, layer["mixer"]), "mixer_norm": norm("norm1"), "mixer_name": "mix.", "feed_forward": ffn,
            "ffn_norm": norm("norm2") if ffn is not None else None, "ffn_name": "mlp.", "mixer_norm_name": "",
            "ffn_norm_name": "", "verbatim_names": True})
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
        # a layer that reads another's keys and values runs on that layer's cache; the first run in the order writes it
        src = layer["mixer"].get("kv_from")
        schedule.append(ScheduleEntry(i, cache=f"kv{i if src is None else src}"))
    e = cfg.embedding
    bigram = e.get("bigram")
    pairs = None if bigram is None else {"name": "bigram", "buckets": int(bigram["buckets"]),
                                         "mul_prev": int(bigram["mul_prev"]), "mul_cur": int(bigram["mul_cur"])}
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=H, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("hashed_bigram_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "embed",
                                                       "suffix": "", "scale": float(e.get("scale", 1.0)), "pairs": pairs}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": "norm", "prefix": "final."}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "head", "suffix": "", "tied_to": None}),
        eos_token_ids=cfg.eos_token_id)
