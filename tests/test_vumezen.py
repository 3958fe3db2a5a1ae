"""The Vumezen design in the engine against the plain implementation (tests/plain_vumezen.py).

Every test makes its own small configuration and weights (tests/vumezen_util.py).  The CPU tests put the plain
PyTorch stand-ins of the kernels (tests/kernel_refs.py) under the engine, so they test what is host logic:
configuration, registry, tensor names, which layers share a cache and how large its window must be, the
previous token as a request's state, batching.  The GPU tests run the same traces on the kernels, in float32
and bfloat16: whole prompts, prompts followed by token-by-token decoding (from CUDA graphs), portions down to
one and two tokens, mixed batches of unequal requests with pages and state slots that are used again, long
prompts whose attention is peaky (a far key, a key at a page's edge, a key one place inside or outside the
window, a kept first token or the one behind them, a stale page would show), heads of the sizes that the
tensor-core kernels take, and greedy generation through ``Engine.generate``.
"""
import copy
import io
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vumezen as P
import replay_util as ru
import vumezen_util as U

DEV = "cuda:0"
# float32: the engine against 64-bit arithmetic, both from the same bfloat16-representable weights, relative to a
# row's largest logit.  bfloat16: products and activations are rounded to 8 bits of mantissa between kernels, and
# the tests' peaky attention (so that a lost key shows) multiplies the rounding of q and k by the scores' spread.
# The float32 runs go through the same kernels and are the sharp test of every index and edge.
TOL = {torch.float32: dict(rtol=5e-5, atol=1e-6), torch.bfloat16: dict(rtol=8e-2, atol=4e-3)}


def make_runner(tmp_path, cfg, weights, dtype, device, **kw):
    from zinfer_b200.engine import ModelRunner

    d = U.write_model(str(tmp_path / f"m{abs(hash(json.dumps(cfg, sort_keys=True))) % 10**8}"), cfg, weights)
    kw.setdefault("page_size", 8)
    kw.setdefault("max_requests", 4)
    return ModelRunner.from_model_dir(d, dtype=dtype, device=device, **kw)


# ============================================================================ CPU
def test_config_is_read_and_registered():
    from zinfer_b200.config import ConfigError, VumezenConfig, family_for, vumezen_model_spec
    from zinfer_b200.engine.model import declared_tensors

    raw = U.CONFIGS["mix"]
    fam = family_for(raw)
    assert fam.name == "Vumezen" and fam.config_class is VumezenConfig
    cfg = VumezenConfig.from_dict(raw)
    assert VumezenConfig.from_dict(cfg.to_dict()) == cfg                      # survives a round trip
    # the tensors the model asks for are exactly the design's names and shapes: a layer that reads another's keys
    # and values has no projections of them, a layer without a feed-forward no second norm
    for name, other in {**U.CONFIGS, **U.MECHANISMS}.items():
        spec = vumezen_model_spec(VumezenConfig.from_dict(other))
        assert {k: tuple(v.shape) for k, v in declared_tensors(spec).items()} == U.tensor_shapes(other), name
    spec = vumezen_model_spec(cfg)
    assert "l1.mix.k" not in declared_tensors(spec) and "l2.norm2" not in declared_tensors(spec)
    # layers 1 and 3 run on the caches of layers 0 and 2
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, "kv0"), (1, "kv0"), (2, "kv2"), (3, "kv2")]
    bad = copy.deepcopy(raw)
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError, match="unknown mixer"):
        VumezenConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][1]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="earlier layer"):
        VumezenConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][3]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError, match="no keys and values of its own"):
        VumezenConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][1]["mixer"]["vdim"] = 8
    with pytest.raises(ConfigError, match="differ"):
        VumezenConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][0]["mlp"]["router"]["top"] = 7
    with pytest.raises(ConfigError, match="cannot be chosen"):
        VumezenConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    bad["layers"][0]["mixer"]["rot"]["dims"] = 18
    with pytest.raises(ConfigError, match="even and at most"):
        VumezenConfig.from_dict(bad)
    bad = copy.deepcopy(raw)
    del bad["embedding"]["bigram"]["mul_prev"]
    with pytest.raises(ConfigError, match="mul_prev"):
        VumezenConfig.from_dict(bad)


def test_command_line_inspects_the_model(tmp_path):
    from zinfer_b200 import cli

    d = U.write_model(str(tmp_path / "m"), U.CONFIGS["mix"], U.make_weights(U.CONFIGS["mix"], seed=1))
    out = io.StringIO()
    assert cli.run(["inspect-config", d], out) == 0
    text = out.getvalue()
    assert "architecture: Vumezen" in text and "token pairs in 53 buckets" in text
    assert "layer 1: attention (heads=4 kv_heads=2 dim=16 vdim=24 scale=0.5 rot dims=8 base=1000.0 window=20 keep_first=1 " \
           "keys and values of layer 0)" in text
    assert "moe experts=6 top=2 scale=1.5 ff=24 shared ff=40" in text and "layer 2: " in text and "feed-forward: none" in text
    out = io.StringIO()
    assert cli.run(["inspect-weights", d], out) == 0 and "tensor_count:" in out.getvalue()


def test_caches_are_shared_and_the_previous_token_is_state():
    from zinfer_b200.config import VumezenConfig, vumezen_model_spec
    from zinfer_b200.engine import DecoderModel

    model = DecoderModel(vumezen_model_spec(VumezenConfig.from_dict(U.CONFIGS["mix"])), torch.float32, "cpu")
    kv, state = model.cache_needs()
    # four layers, two caches; a cache must serve the widest window and the most kept tokens among its readers
    assert sorted(kv) == ["kv0", "kv2"]
    assert (kv["kv0"].window, kv["kv0"].keep_first) == (20, 3) and (kv["kv2"].window, kv["kv2"].keep_first) == (12, 6)
    assert all(n.num_kv_heads == 2 and n.head_dim == 16 and n.value_dim == 24 and n.values for n in kv.values())
    # one 32-bit integer per request: its last token
    assert list(state) == ["embedding"] and state["embedding"].shape == (1,) and state["embedding"].dtype == torch.int32
    model = DecoderModel(vumezen_model_spec(VumezenConfig.from_dict(U.CONFIGS["alt"])), torch.float32, "cpu")
    kv, state = model.cache_needs()
    assert sorted(kv) == ["kv0", "kv1"] and kv["kv0"].value_dim == 16 and kv["kv1"].value_dim in (None, 8)


def test_weights_of_wrong_shape_are_refused(tmp_path):
    from zinfer_b200.engine import ModelRunner

    cfg = U.CONFIGS["odd"]
    w = U.make_weights(cfg, seed=2)
    w["l0.mix.v"] = torch.zeros(10, 44, dtype=torch.bfloat16)            # values of the keys' size, not their own
    d = U.write_model(str(tmp_path / "bad"), cfg, w)
    with pytest.raises(Exception, match="l0.mix.v"):
        ModelRunner.from_model_dir(d, dtype=torch.float32, device="cpu", page_size=8, max_tokens=64, max_requests=2,
                                   cuda_graphs=False)
    w = U.make_weights(cfg, seed=2)
    w["l1.mix.k"] = torch.zeros(10, 44, dtype=torch.bfloat16)            # a reader of another layer's keys has none
    d = U.write_model(str(tmp_path / "extra"), cfg, w)
    with pytest.raises(Exception, match="l1.mix.k"):
        ModelRunner.from_model_dir(d, dtype=torch.float32, device="cpu", page_size=8, max_tokens=64, max_requests=2,
                                   cuda_graphs=False)


@pytest.mark.parametrize("name", ["mix", "alt", "odd"])
def test_engine_host_logic_on_stand_ins(cpu_kernels, tmp_path, name):
    cfg = U.CONFIGS[name]
    weights = U.make_weights(cfg, seed=3)
    runner = make_runner(tmp_path, cfg, weights, torch.float32, "cpu", max_tokens=192, max_requests=3, cuda_graphs=False)
    reqs = ru.make_requests(cfg["vocab"], [23, 1, 40, 9, 17], seed=4)
    plain = U.plain_logits(cfg, weights, reqs)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 6)),
                        ("portions", ru.trace_portions(reqs, 2)), ("mixed", ru.trace_mixed(reqs, 5, max_live=3, tail=4))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, rtol=2e-4, atol=1e-5)
        assert not runner.manager.requests
    assert runner.manager.slots.reused > 0            # three slots served five requests, four times over


def test_plain_model_pieces():
    """The plain implementation against numbers worked out by hand."""
    F = torch.float64
    # the pair table: row (previous * 3 + token * 5) mod 7, the last row at a sequence's start
    e = {"scale": 2.0, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}}
    assert [P.bigram_row(None, 4, e), P.bigram_row(6, 4, e), P.bigram_row(0, 0, e)] == [7, (18 + 20) % 7, 0]
    w = {"embed": torch.arange(10, dtype=F).reshape(5, 2), "bigram": 100.0 * torch.arange(16, dtype=F).reshape(8, 2)}
    x = P.embed([4, 1], None, w, e)
    assert x.tolist() == [[16.0 + 1400.0, 18.0 + 1500.0], [4.0 + 200.0 * ((12 + 5) % 7), 6.0 + 100.0 * (2 * ((12 + 5) % 7) + 1)]]
    # rotation of the first two of three dimensions: (1, 0) at position 1 with base 1 -> (cos 1, sin 1); the third passes
    r = P.rotate(torch.tensor([[[1.0, 0.0, 7.0]]], dtype=F), torch.tensor([1]), 2, 1.0)
    assert torch.allclose(r, torch.tensor([[[np.cos(1.0), np.sin(1.0), 7.0]]], dtype=F))
    # the second pair of four rotates by position * base^(-2/4)
    r = P.rotate(torch.tensor([[[0.0, 1.0, 0.0, 0.0]]], dtype=F), torch.tensor([3]), 4, 16.0)
    assert torch.allclose(r, torch.tensor([[[0.0, np.cos(0.75), 0.0, np.sin(0.75)]]], dtype=F))
    # the mask: a window of 3 that keeps 2 first tokens, seen from position 6
    assert [j for j in range(9) if P.visible(6, j, 3, 2)] == [0, 1, 4, 5, 6]
    assert [j for j in range(9) if P.visible(1, j, 3, 2)] == [0, 1] and [j for j in range(9) if P.visible(6, j, 1, 0)] == [6]
    # the sink: one key of score 0 gets weight 1/2, so the output is half its value
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 3, "scale": 1.0, "mask": {"size": 4, "keep_first": 0},
         "rot": {"dims": 2, "base": 10.0}}
    p = {"q": torch.zeros(2, 2, dtype=F), "o": torch.eye(3, dtype=F)}
    out = P.attend(torch.ones(1, 2, dtype=F), p, m, 0, torch.ones(1, 1, 2, dtype=F), torch.tensor([[[2.0, 4.0, 6.0]]], dtype=F))
    assert torch.allclose(out, torch.tensor([[1.0, 2.0, 3.0]], dtype=F))
    # routing: scores 0.6, 0.5, 0.4; the correction lifts the last above the second; weights stay scores times the scale
    logit = lambda s: float(np.log(s / (1 - s)))
    pw = {"router": torch.tensor([[logit(0.6)], [logit(0.5)], [logit(0.4)]], dtype=F), "correction": torch.tensor([0.0, 0.0, 0.2], dtype=F)}
    for e_ in range(3):
        pw[f"e{e_}.up"] = torch.tensor([[float(e_ + 1)]], dtype=F)
        pw[f"e{e_}.down"] = torch.tensor([[1.0]], dtype=F)
    mlp = {"router": {"experts": 3, "top": 2, "scale": 2.0}, "expert": {"ff": 1}}
    assert P.choose(torch.tensor([0.6, 0.5, 0.4], dtype=F), pw["correction"], 2) == [2, 0] or \
        sorted(P.choose(torch.tensor([0.6, 0.5, 0.4], dtype=F), pw["correction"], 2)) == [0, 2]
    out = P.moe(torch.ones(1, 1, dtype=F), pw, mlp)                     # experts square their input times 1 and 3
    assert abs(out.item() - 2.0 * (0.6 * 1.0 + 0.4 * 9.0)) < 1e-12
    assert abs(P.relu2_expert(torch.tensor([[-1.0]], dtype=F), pw["e0.up"], pw["e0.down"]).item()) == 0.0


# ============================================================================ GPU
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(U.MECHANISMS))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = U.MECHANISMS[name]
    weights = U.make_weights(cfg, seed=11)
    reqs = U.clear_requests(cfg, weights, [37, 1, 20], seed=12, margin=0.05)
    plain = U.plain_logits(cfg, weights, reqs)
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=128, max_requests=2)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 12)),
                        ("portions", ru.trace_portions(reqs, 7, sizes=(2, 1, 5, 2, 3, 9, 2)))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, **TOL[dtype])
    runner.manager.check()


@pytest.fixture(scope="module")
def models():
    """Per configuration: weights, requests with clear choices of experts, the plain model's logits."""
    out = {}
    for name, cfg in U.CONFIGS.items():
        weights = U.make_weights(cfg, seed=21 + len(name))
        reqs = U.clear_requests(cfg, weights, [45, 3, 70, 18, 1, 33], seed=5, margin=0.04)
        out[name] = (cfg, weights, reqs, U.plain_logits(cfg, weights, reqs))
    return out


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(U.CONFIGS))
def test_whole_decode_portions_mixed(tmp_path, models, name, dtype):
    cfg, weights, reqs, plain = models[name]
    # pool: the three longest requests rounded up to pages, so pages and the three slots are used again
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=176, max_requests=3, poison_freed_pages=True)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 24)),
                        ("portions", ru.trace_portions(reqs, 9)), ("mixed", ru.trace_mixed(reqs, 13, max_live=3, tail=10))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"{name}/{mode}", argmax_frac=0.0, **TOL[dtype])
        assert not runner.manager.requests
    assert runner.graphs is not None and runner.graphs.replays > 0         # single tokens came from CUDA graphs
    assert sum(g.pool.reused for g in runner.manager.groups) > 0
    assert runner.manager.slots.reused > 0
    runner.manager.check()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batch_against_each_alone(tmp_path, models, dtype):
    """Unequal requests in one batch give the rows they give alone, to the last bits in float32."""
    from zinfer_b200.engine import StepEntry

    cfg, weights, reqs, _ = models["mix"]
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=256, max_requests=4)
    ids = ["r0", "r2", "r3", "r4"]
    alone = {}
    for rid in ids:
        alone[rid] = runner.step([StepEntry(rid, reqs[rid], list(range(len(reqs[rid]))))]).clone()
        runner.end_request(rid)
    # together: the first request has half of its tokens in the cache already, the others come whole
    half = len(reqs["r0"]) // 2
    runner.step([StepEntry("r0", reqs["r0"][:half], [])])
    entries = [StepEntry("r0", reqs["r0"][half:], list(range(len(reqs["r0"]) - half)))] + \
        [StepEntry(rid, reqs[rid], list(range(len(reqs[rid])))) for rid in ids[1:]]
    got = runner.step(entries)
    row = 0
    for e in entries:
        want = alone[e.request_id][-len(e.want):]
        part = got[row:row + len(e.want)]
        row += len(e.want)
        tol = 2e-6 if dtype == torch.float32 else 2e-2
        assert (part - want).abs().max() <= tol * want.abs().max(), e.request_id


MARKER = 7          # the token whose key every query prefers (see _marked)


def _marked(dim, vdim, heads, kv_heads, window, keep, reader_window, reader_keep):
    """Two attention layers without feed-forwards (the second reads the first's cache, with a mask of its own) and
    weights in which one token's key stands out: every token's embedding has the same positive first coordinate, the
    token MARKER's is eight times larger, and one unrotated coordinate of every query and key head reads it.  A query
    that sees a MARKER gives it nearly all of its softmax; the table of token pairs makes two MARKERs' values differ."""
    a = U.att(heads, kv_heads, dim, vdim, 1.5 / dim ** 0.5, window, keep, rot_dims=dim // 2, base=2000.0)
    b = {**a, "mask": {"size": reader_window, "keep_first": reader_keep}, "kv_from": 0}
    cfg = U.config(149, 96, [U.layer(a, None), U.layer(b, None)], scale=2.0, bigram=(29, 7, 3))
    w = U.make_weights(cfg, seed=31)
    w["embed"][:, 0] = 1.0
    w["embed"][MARKER, 0] = 8.0
    w["bigram"][:, 0] = 0.0
    gain = (2.0 * dim ** 0.5) ** 0.5          # a MARKER's score leads the others' by about 9
    for name, n in (("l0.mix.q", heads), ("l0.mix.k", kv_heads), ("l1.mix.q", heads)):
        for h in range(n):
            w[name][h * dim + dim - 1, 0] = gain
    for name in ("l0.mix.o", "l1.mix.o"):            # what the mixers add weighs as much as the embedding
        w[name] = (w[name].float() * 4.0).to(torch.bfloat16)
    return cfg, w


def _marked_request(vocab, length, marks, seed):
    toks = [t if t != MARKER else MARKER + 1 for t in ru.make_requests(vocab, [length], seed)["r0"]]
    for p in marks:
        if 0 <= p < length:
            toks[p] = MARKER
    return toks


def _wrong_masks(cfg, weights, reqs):
    """The plain model's logits with a mask that is off by one at each edge, and without the sink: what an engine
    with that fault would give."""
    out = {}
    right = P.visible
    variants = {
        "window one too wide": lambda i, j, size, keep: right(i, j, size + 1, keep),
        "window one too narrow": lambda i, j, size, keep: right(i, j, size - 1, keep),
        "one kept token too few": lambda i, j, size, keep: right(i, j, size, max(0, keep - 1)),
        "one kept token too many": lambda i, j, size, keep: right(i, j, size, keep + 1),
    }
    try:
        for what, fn in variants.items():
            P.visible = fn
            out[what] = U.plain_logits(cfg, weights, reqs)
        P.visible = right
        P.SINK = 0.0
        out["no sink"] = U.plain_logits(cfg, weights, reqs)
    finally:
        P.visible = right
        P.SINK = 1.0
    return out


EDGE_CASES = [
    (16, 24, 4, 2, 21, 3, 8),        # the general kernels in both types; the window's edge moves through pages of 8
    (64, 64, 4, 1, 50, 5, 16),       # heads the tensor-core kernels take in bfloat16; a window shorter than their key tiles
    (128, 128, 2, 2, 150, 70, 32),   # more kept tokens than a tile of keys; a window of several tiles
    (64, 32, 2, 1, 33, 1, 16),       # values half the keys' size
]


def _edge_case(dim, vdim, heads, kv_heads, window, keep):
    """Configuration, weights, requests and the plain logits of a case whose MARKERs stand at the last kept place and
    the one behind it, and where the window's edge passes them in the prompt and again among the decoded tokens."""
    cfg, weights = _marked(dim, vdim, heads, kv_heads, window, keep, reader_window=window + 7, reader_keep=max(1, keep - 1))
    n = 2 * window + keep + 60
    reqs = {"r0": _marked_request(cfg["vocab"], n, [keep - 1, keep, keep + 12, window + keep + 25], seed=6),
            "r1": _marked_request(cfg["vocab"], window + keep + 2, [0, keep, keep + 1], seed=7),
            "r2": _marked_request(cfg["vocab"], keep + 1, [keep - 1, keep], seed=8),
            "r3": _marked_request(cfg["vocab"], 3, [1], seed=9)}
    return cfg, weights, reqs, U.plain_logits(cfg, weights, reqs)


@pytest.mark.parametrize("dim,vdim,heads,kv_heads,window,keep,page", EDGE_CASES[:1] + EDGE_CASES[3:])
def test_the_marked_requests_show_every_fault_of_the_mask(dim, vdim, heads, kv_heads, window, keep, page):
    """The plain model alone: with a window one key wider or narrower, one kept token more or fewer, or no sink, the
    logits of the marked requests move by far more than the loosest tolerance of the tests below, in the part that those
    tests run both as a prompt and token by token."""
    cfg, weights, reqs, plain = _edge_case(dim, vdim, heads, kv_heads, window, keep)
    n = len(reqs["r0"])
    tail = n - (window + keep + 50)
    for what, other in _wrong_masks(cfg, weights, {"r0": reqs["r0"]}).items():
        moved = np.abs(other["r0"] - plain["r0"]).max(axis=-1) / np.abs(plain["r0"]).max(axis=-1)
        limit = 4 * TOL[torch.bfloat16]["rtol"]
        if what != "no sink":                      # (these requests' scores are large: the sink has a test of its own)
            assert (moved[tail:] > limit).sum() >= 1, (what, moved.max())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,vdim,heads,kv_heads,window,keep,page", EDGE_CASES)
def test_every_edge_of_the_mask_decides(tmp_path, dtype, dim, vdim, heads, kv_heads, window, keep, page):
    """Prompts of hundreds of tokens in which one token's key stands out, placed at every edge of the mask (the test
    above shows that each fault of the mask moves these logits by far more than the tolerance).  The engine must match
    the right mask: whole, in portions that end around page edges, decoding token by token far past the window (so
    that every page but the first leaves it), and mixed."""
    cfg, weights, reqs, plain = _edge_case(dim, vdim, heads, kv_heads, window, keep)
    n = len(reqs["r0"])
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=page, max_tokens=2 * (n + page) + 4 * page,
                         max_requests=3, poison_freed_pages=True)
    edges = (page, page - 1, 1, page + 1, 2 * page - 1, 2, window, 2, window - 1, 3, window + 1, 1, 1, 5)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("edges", ru.trace_portions(reqs, 0, sizes=edges)),
                        ("long decode", ru.trace_tail_decode(reqs, window + keep + 50)),
                        ("mixed", ru.trace_mixed(reqs, 3, max_live=3, tail=window + 9))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"edges {dim}/{vdim}/{mode}", argmax_frac=0.0, **TOL[dtype])
    assert runner.graphs is not None and runner.graphs.replays > window
    runner.manager.check()


@gpu
def test_the_sink_carries_the_first_tokens(tmp_path):
    """With small scores the sink holds a large share of the softmax's denominator, most of all at a sequence's first
    tokens: the plain model without it gives other logits by far, and the engine matches the one with it, in prompts,
    in portions and in decoding, by the general kernels and (heads of 64, bfloat16) by the tensor-core kernels."""
    for dim in (8, 64):
        cfg = U.config(61, 32, [U.layer(U.att(2, 1, dim, dim, 0.3 / dim ** 0.5, 6, 1, rot_dims=4), None)], scale=1.0, bigram=None)
        weights = U.make_weights(cfg, seed=61)
        weights["l0.mix.o"] = (weights["l0.mix.o"].float() * 8.0).to(torch.bfloat16)
        reqs = ru.make_requests(cfg["vocab"], [12, 2, 1], seed=9)
        plain = U.plain_logits(cfg, weights, reqs)
        P.SINK = 0.0
        try:
            no_sink = U.plain_logits(cfg, weights, reqs)
        finally:
            P.SINK = 1.0
        assert all(np.abs(plain[r] - no_sink[r]).max() > 0.1 * np.abs(plain[r]).max() for r in reqs)
        for dtype in (torch.float32, torch.bfloat16):
            runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
            for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 11), ru.trace_portions(reqs, 3, sizes=(2, 1, 2, 3))):
                ru.assert_close(ru.run_in_process(runner, trace), plain, what="sink", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_a_single_far_key_decides(tmp_path):
    """One key hundreds of tokens back (no window is left here) carries much of the last query's softmax: among all
    tokens that could stand at position 19, the test takes the one whose presence moves the last position's logits most
    in the plain model, and requires that move to be large; an engine that lost that key could not match."""
    cfg = U.config(67, 32, [U.layer(U.att(2, 1, 8, 12, 1.5, 1000, 0, rot_dims=4, base=100.0), None)], scale=1.0, bigram=None)
    weights = U.make_weights(cfg, seed=41)
    toks = ru.make_requests(cfg["vocab"], [270], seed=7)["r0"]
    without = toks[:19] + [toks[18]] + toks[20:]
    lost = U.plain_logits(cfg, weights, {"r0": without})
    move = {c: np.abs(U.plain_logits(cfg, weights, {"r0": toks[:19] + [c] + toks[20:]})["r0"][-1] - lost["r0"][-1]).max()
            for c in range(cfg["vocab"])}
    toks[19] = max(move, key=move.get)
    plain = U.plain_logits(cfg, weights, {"r0": toks})
    assert np.abs(plain["r0"][-1] - lost["r0"][-1]).max() > 0.05 * np.abs(plain["r0"][-1]).max()     # the far key matters
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=288, max_requests=1)
        for trace in (ru.trace_whole({"r0": toks}), ru.trace_tail_decode({"r0": toks}, 5)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="one far key", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_the_previous_token_survives_portions_and_slots(tmp_path):
    """The pair table is made as large as everything else together, so a wrong previous token (lost at the start of a
    portion, taken from another request's slot, or not reset when a slot is used again) changes every logit."""
    cfg = U.config(61, 32, [U.layer(U.att(2, 1, 8, 8, 0.1, 5, 0), None)], scale=1.0, bigram=(13, 5, 3))
    weights = U.make_weights(cfg, seed=51)
    reqs = ru.make_requests(cfg["vocab"], [9, 4, 1, 14, 6, 2, 11], seed=8)
    plain = U.plain_logits(cfg, weights, reqs)
    # the plain model that forgets the previous token at every call differs from the second token on
    forgetful = P.PlainVumezen(cfg, weights)
    a = forgetful.forward(reqs["r0"][:4])
    forgetful.prev = None
    b = forgetful.forward(reqs["r0"][4:])
    assert np.abs(b.numpy()[0] - plain["r0"][4]).max() > 0.2 * np.abs(plain["r0"][4]).max() and np.allclose(a.numpy(), plain["r0"][:4])
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
        for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 5), ru.trace_portions(reqs, 1, sizes=(2, 1, 3, 2)),
                      ru.trace_mixed(reqs, 2, max_live=2, tail=3)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="previous token", argmax_frac=0.0, **TOL[dtype])
        assert runner.manager.slots.reused > 0


@gpu
def test_the_correction_changes_choices_but_not_weights(tmp_path):
    """In the plain model some tokens' chosen experts differ with and without the correction; the engine matches the one
    with it, and the weights are the uncorrected scores (a model whose weights took the correction would differ)."""
    cfg = U.MECHANISMS["experts"]
    weights = U.make_weights(cfg, seed=61)
    reqs = U.clear_requests(cfg, weights, [40, 7], seed=9, margin=0.05)
    plain = U.plain_logits(cfg, weights, reqs)
    zero = {**weights, "l0.mlp.correction": torch.zeros_like(weights["l0.mlp.correction"])}
    assert np.abs(U.plain_logits(cfg, zero, reqs)["r0"] - plain["r0"]).max() > 0.05 * np.abs(plain["r0"]).max()
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
        for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 9)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="correction", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_greedy_generation_through_the_engine(tmp_path, models):
    from zinfer_b200.engine.api import Engine
    from zinfer_b200.sampling import SamplingParams

    cfg, weights, reqs, _ = models["mix"]
    d = U.write_model(str(tmp_path / "gen"), cfg, weights)
    prompts = [reqs["r1"], reqs["r3"], reqs["r0"][:30], reqs["r4"]]
    eng = Engine(d, dtype="float32", device=DEV, page_size=8, kv_cache_tokens=192, max_batched_tokens=16, max_requests=3)
    got = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=25, ignore_eos=True))
    for p, r in zip(prompts, got):
        assert len(r.token_ids) == 25                              # past the windows of 12 and 20 tokens
        logits = P.PlainVumezen(cfg, weights).forward(p + r.token_ids).numpy()
        for i, t in enumerate(r.token_ids):      # the best token given the same history, or tied with it to rounding
            row = logits[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-4 * np.abs(row).max()


@gpu
def test_command_line_makes_a_random_model_and_generates(tmp_path):
    """bin/zinfer: a model folder of random weights made from a Vumezen config.json, then tokens from it, greedy and sampled."""
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(U.CONFIGS["odd"]))
    d = str(tmp_path / "random")
    tool = os.path.join(ru.REPO, "bin", "zinfer")
    r = subprocess.run([sys.executable, tool, "random-model", d, str(cfg_path), "7"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    r = subprocess.run([sys.executable, tool, "generate-token-ids", d, "5,17,3,60,2", "6", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tokens: [5, 17, 3, 60, 2, " in r.stdout, r.stderr[-2000:]
    r = subprocess.run([sys.executable, tool, "generate-token-ids", d, "5,17,3,60,2", "6", "--temperature", "0.8", "--top-k", "10",
                        "--seed", "3"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tokens: [5, 17, 3, 60, 2, " in r.stdout, r.stderr[-2000:]


@gpu
def test_replay_program(tmp_path, models):
    """bin/trace_run as a user runs it: the model class comes from config.json, four state slots."""
    cfg, weights, reqs, plain = models["odd"]
    d = U.write_model(str(tmp_path / "tool"), cfg, weights)
    trace = ru.trace_mixed(reqs, 3, max_live=4, tail=8)
    info = {}
    got = ru.run_trace_tool(d, "float32", trace, str(tmp_path / "out"), ru.max_live_tokens(trace), cfg["vocab"], info=info)
    ru.assert_close(got, plain, what="trace_run", argmax_frac=0.0, **TOL[torch.float32])
    assert info["pages_reused"] and info["pages_reused"] > 0
