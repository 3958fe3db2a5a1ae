"""Typed configuration of the Sepitar design and its model spec.

A Sepitar model is a decoder whose layers norm the stream ONCE and add both sublayers' outputs to it:
with n = norm1(x), x <- x + mixer(n) + ff(n); the norm's stored weight lies around zero (the multiplier is 1 + w).
A layer's ``type`` names its mixer:

* ``attention``: grouped-query attention with biases on q, k, v and the output projection, no rotation, a learned
  bias per head and distance bucket (``rel`` [rows, heads]; ``bias_max`` is where the logarithmic buckets end), a
  sliding window ``mask.size``, a plain softmax, and an output gate per channel, sigmoid(W_g n).
* ``attention_2``: no biases; an RMS norm over ALL of q and all of k (plain weights) before the heads are split;
  rotation of the first ``rot.dims`` dimensions of every head in pairs (i, i + dims/2) with the frequencies rescaled
  by wavelength (``rot.scaling``: factor, low, high, original); the score is capped, c tanh(s / c) with c =
  ``softcap``; every earlier key is visible; a learned sink per head joins the softmax's denominator; an output gate
  per head.
* ``latent_attention``: queries through a normed latent of ``q_rank`` values; per token one normed latent of
  ``kv_rank`` values, from which every head's unrotated keys and its values are linear maps, plus ``rot_dim``
  rotated key values shared by all heads; rotation in pairs (2i, 2i + 1) with ramped frequency scaling
  (``rot.scaling``: factor, original, fast, slow) and its magnitude factor; a sliding window; a learned sink.

The feed-forward is a mixture of clamped gated experts (router logits with a bias, the ``top`` largest chosen, weights
= the softmax over the chosen) beside a shared expert, or absent.  ``loop`` {start, stop, times} runs layers start ..
stop - 1 ``times`` times in a row, every pass with caches of its own; before every pass but the first the embedding's
output is added to the stream.  config.json gives every size and every constant that may differ between models; the
tensor names (``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``) are fixed, and so
are the experts' gate g sigmoid(1.702 g) (u + 1) and the one added to the norms' weights.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Optional

from .luvavik import _positive
from .qwen3 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Sepitar"
DEFAULT_MAX_POSITIONS = 1 << 17       # the design has no position limit; the engine needs one for its tables
ACT_ALPHA = 1.702                     # the experts' gate is g * sigmoid(ACT_ALPHA * g): fixed by the design

MIXERS = ("attention", "attention_2", "latent_attention")


def _mask_ok(where: str, m: dict) -> None:
    mask = m.get("mask")
    if mask is not None:
        _positive(f"{where}.mask", mask, ("size",))


def _rot_ok(where: str, m: dict, limit: int, scaling_keys: tuple) -> None:
    rot = m.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where} lacks its rotation")
    _positive(f"{where}.rot", rot, ("base", "dims"))
    if rot["dims"] % 2 or rot["dims"] > limit:
        raise ConfigError(f"config.json: {where}.rot.dims {rot['dims']} must be even and at most {limit}")
    if rot.get("scaling") is not None:
        _positive(f"{where}.rot.scaling", rot["scaling"], scaling_keys)


@dataclass(frozen=True)
class SepitarConfig:
    vocab_size: int
    hidden_size: int
    layers: tuple[dict, ...]               # as in config.json: type, mixer, mlp
    norm_eps: float
    loop: Optional[dict] = None            # start, stop, times
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_id: tuple[int, ...] = field(default_factory=tuple)
    model_type: str = "sepitar"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "SepitarConfig":
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
                  loop=copy.deepcopy(d.get("loop")) or None,
                  max_position_embeddings=int(d.get("max_position_embeddings", DEFAULT_MAX_POSITIONS)),
                  eos_token_id=tuple(int(t) for t in (eos or ())))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ConfigError("vocab and width must be positive")
        if not self.norm_eps >= 0.0:
            raise ConfigError(f"norm.eps must be >= 0, got {self.norm_eps}")
        if self.loop is not None:
            for k in ("start", "stop", "times"):
                if not isinstance(self.loop.get(k), int):
                    raise ConfigError(f"config.json: loop lacks the integer {k!r}")
            if not 0 <= self.loop["start"] < self.loop["stop"] <= len(self.layers) or self.loop["times"] < 1:
                raise ConfigError(f"config.json: loop {self.loop} does not name a range of the {len(self.layers)} layers run at least once")
        for i, layer in enumerate(self.layers):
            kind, m = layer.get("type"), layer.get("mixer")
            if kind not in MIXERS:
                raise ConfigError(f"config.json: layer {i} has the unknown mixer type {kind!r}; known: {', '.join(MIXERS)}")
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: layer {i} lacks its mixer's sizes")
            where = f"layers[{i}].mixer"
            _mask_ok(where, m)
            if kind == "latent_attention":
                _positive(where, m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"))
                _rot_ok(where, m, m["rot_dim"], ("factor", "original", "fast", "slow"))
            else:
                _positive(where, m, ("heads", "kv_heads", "dim", "vdim", "scale"))
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {where}: {m['heads']} heads do not divide into {m['kv_heads']} kv heads")
                if kind == "attention":
                    _positive(where, m, ("bias_max",))
                else:
                    _positive(where, m, ("softcap",))
                    _rot_ok(where, m, m["dim"], ("factor", "low", "high", "original"))
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind", "moe") != "moe":
                raise ConfigError(f"config.json: layer {i} has the unknown feed-forward kind {mlp.get('kind')!r}; known: moe")
            _positive(f"layers[{i}].mlp.expert", mlp.get("expert") or {}, ("ff", "limit"))
            router = mlp.get("router") or {}
            _positive(f"layers[{i}].mlp.router", router, ("experts", "top"))
            if router["top"] > router["experts"]:
                raise ConfigError(f"config.json: layer {i}: {router['top']} of {router['experts']} experts cannot be chosen")
            if mlp.get("shared") is not None:
                _positive(f"layers[{i}].mlp.shared", mlp["shared"], ("ff", "limit"))

    def runs(self) -> list[tuple[int, int, bool]]:
        """(layer, pass, first run of a pass after the first) in the order in which the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, 0, False) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        out = [(i, 0, False) for i in range(a)]
        for p in range(times):
            out += [(i, p, p > 0 and i == a) for i in range(a, b)]
        return out + [(i, 0, False) for i in range(b, n)]

    def describe(self) -> list[str]:
        """Lines for the command line's model inspection."""
        lines = [f"hidden_size: {self.hidden_size}", f"vocab_size: {self.vocab_size}", f"num_layers: {len(self.layers)}",
                 f"layer_runs: {len(self.runs())}", f"norm_eps: {self.norm_eps:e}"]
        if self.loop is not None:
            lines.append(f"loop: layers {self.loop['start']}..{self.loop['stop'] - 1} run {self.loop['times']} times")
        for i, layer in enumerate(self.layers):
            m, kind = layer["mixer"], layer["type"]
            mask = m.get("mask")
            window = f" window={mask['size']}" if mask else " no window"
            if kind == "latent_attention":
                mixer = (f"heads={m['heads']} dim={m['dim']} rot_dim={m['rot_dim']} vdim={m['vdim']} q_rank={m['q_rank']} "
                         f"kv_rank={m['kv_rank']} scale={m['scale']}{window}")
            else:
                mixer = (f"heads={m['heads']} kv_heads={m['kv_heads']} dim={m['dim']} vdim={m['vdim']} scale={m['scale']}"
                         + (f" bias_max={m['bias_max']}{window}" if kind == "attention" else f" softcap={m['softcap']} rot dims={m['rot']['dims']}"))
            mlp = layer.get("mlp")
            if mlp is None:
                ff = "none"
            else:
                r = mlp["router"]
                ff = (f"moe experts={r['experts']} top={r['top']} ff={mlp['expert']['ff']} limit={mlp['expert']['limit']}"
                      + (f" shared ff={mlp['shared']['ff']} limit={mlp['shared']['limit']}" if mlp.get("shared") else ""))
            lines.append(f"layer {i}: {kind} ({mixer}); feed-forward: {ff}")
        return lines

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                             "layers": [copy.deepcopy(layer) for layer in self.layers], "norm": {"eps": self.norm_eps}}
        if self.loop is not None:
            d["loop"] = copy.deepcopy(self.loop)
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d


# ---------------------------------------------------------------------- the family
def _rope(cfg: SepitarConfig, rot: dict, kind: str, pairing: str) -> PartSpec:
    scaling = None
    if rot.get("scaling") is not None:
        scaling = {"kind": kind, **{k: float(v) for k, v in rot["scaling"].items()}}
    return PartSpec("rope", {"head_dim": int(rot["dims"]), "theta": float(rot["base"]), "scaling": scaling, "pairing": pairing,
                             "max_positions": cfg.max_position_embeddings})


def _mixer_spec(cfg: SepitarConfig, kind: str, m: dict) -> PartSpec:
    H = cfg.hidden_size
    mask = m.get("mask")
    window = int(mask["size"]) if mask else None
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": H, "num_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
            "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]), "scale": float(m["scale"]),
            "norm_eps": cfg.norm_eps, "window": window, "learned_sink": True, "output_gate": False,
            "position": _rope(cfg, m["rot"], "ramp", "neighbours")})
    common = {"hidden_size": H, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
              "value_dim": int(m["vdim"]), "qk_norm_eps": None, "scale": float(m["scale"]), "window": window,
              "names": {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "sink": "sink"}}
    if kind == "attention":
        return PartSpec("gqa_attention", {**common, "position": None, "bias": True, "output_gate": "channel",
                                          "distance_bias": {"rows": None, "far": float(m["bias_max"]), "name": "rel"}})
    return PartSpec("gqa_attention", {**common, "position": _rope(cfg, m["rot"], "by_wavelength", "halves"),
                                      "whole_norm_eps": cfg.norm_eps, "softcap": float(m["softcap"]), "learned_sink": True,
                                      "output_gate": "head"})


def _expert(H: int, e: dict) -> PartSpec:
    return PartSpec("swiglu_mlp", {"hidden_size": H, "intermediate_size": int(e["ff"]), "activation": "clamped_gated",
                                   "limit": float(e["limit"]), "act_alpha": ACT_ALPHA, "names": ("gate", "up", "down")})


def _ffn_spec(cfg: SepitarConfig, layer: dict) -> Optional[PartSpec]:
    mlp = layer.get("mlp")
    if mlp is None:
        return None
    H = cfg.hidden_size
    router = mlp["router"]
    return PartSpec("routed_experts", {
        "hidden_size": H, "intermediate_size": int(mlp["expert"]["ff"]), "experts": int(router["experts"]),
        "top": int(router["top"]), "score": "top_logits", "router_bias": True, "activation": "clamped_gated",
        "limit": float(mlp["expert"]["limit"]), "act_alpha": ACT_ALPHA, "expert_names": "e{}.", "gate_name": "gate",
        "shared": _expert(H, mlp["shared"]) if mlp.get("shared") is not None else None, "shared_name": "shared."})


def sepitar_model_spec(cfg: SepitarConfig) -> ModelSpec:
    H = cfg.hidden_size
    norm = lambda tensor: PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": tensor, "one_plus": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        block = PartSpec("parallel_block", {
            "mixer": _mixer_spec(cfg, layer["type"], layer["mixer"]), "mixer_norm": norm("norm1"), "mixer_name": "mix.",
            "feed_forward": _ffn_spec(cfg, layer), "ffn_norm": None, "ffn_name": "mlp.", "mixer_norm_name": "",
            "ffn_norm_name": "", "verbatim_names": True})
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    # every run has a cache of its own (no name: the model gives each its own); the first run of every further pass
    # takes the embedding's output in again
    schedule = tuple(ScheduleEntry(i, pre_add_input=again) for i, _, again in cfg.runs())
    return ModelSpec(
        architecture=ARCHITECTURE, vocab_size=cfg.vocab_size, hidden_size=H, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "embed", "suffix": ""}),
        layers=tuple(layers), schedule=schedule,
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.norm_eps, "tensor": "norm", "prefix": "final.", "one_plus": True}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": H, "name": "head", "suffix": "", "tied_to": None}),
        eos_token_ids=cfg.eos_token_id)
