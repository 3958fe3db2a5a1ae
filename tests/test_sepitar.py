"""The Sepitar design in the engine against the plain implementation (tests/plain_sepitar.py).

Every test makes its own small configuration and weights (tests/sepitar_util.py).  The CPU tests put the plain
PyTorch stand-ins of the kernels (tests/kernel_refs.py) under the engine, so they test what is host logic:
configuration, registry, tensor names, the order of layer runs and their caches, batching.  The GPU tests run the
same traces on the kernels, in float32 and bfloat16: every mechanism alone, whole prompts, prompts followed by
token-by-token decoding (from CUDA graphs), portions down to one and two tokens, mixed batches of unequal requests
with pages and state slots that are used again, long prompts with peaky attention (a far key, a key one place
inside or outside the window, a sink that carries the first tokens, a distance table that decides), and greedy
generation through ``Engine.generate``.
"""
import copy
import io
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_sepitar as P
import replay_util as ru
import sepitar_util as U

DEV = "cuda:0"
# float32: the engine against 64-bit arithmetic, both from the same bfloat16-representable weights, relative to a
# row's largest logit.  bfloat16: products and activations are rounded to 8 bits of mantissa between kernels, and
# the tests' peaky attention (so that a lost key shows) multiplies the rounding of q and k by the scores' spread.
TOL = {torch.float32: dict(rtol=5e-5, atol=1e-6), torch.bfloat16: dict(rtol=8e-2, atol=4e-3)}


def make_runner(tmp_path, cfg, weights, dtype, device, **kw):
    from zinfer_b200.engine import ModelRunner

    d = U.write_model(str(tmp_path / f"m{abs(hash(json.dumps(cfg, sort_keys=True))) % 10**8}"), cfg, weights)
    kw.setdefault("page_size", 8)
    kw.setdefault("max_requests", 4)
    return ModelRunner.from_model_dir(d, dtype=dtype, device=device, **kw)


# ============================================================================ CPU
def test_config_is_read_and_registered():
    from zinfer_b200.config import ConfigError, SepitarConfig, family_for, sepitar_model_spec
    from zinfer_b200.engine.model import declared_tensors

    raw = U.public(U.CONFIGS["mix"])
    fam = family_for(raw)
    assert fam.name == "Sepitar" and fam.config_class is SepitarConfig
    cfg = SepitarConfig.from_dict(raw)
    assert SepitarConfig.from_dict(cfg.to_dict()) == cfg                      # survives a round trip
    # the tensors the model asks for are exactly the design's names and shapes; the distance table's rows are free
    for name, other in {**U.CONFIGS, **U.MECHANISMS}.items():
        spec = sepitar_model_spec(SepitarConfig.from_dict(U.public(other)))
        declared = declared_tensors(spec)
        want = U.tensor_shapes(other)
        assert set(declared) == set(want), name
        assert all(declared[k].fits(want[k]) for k in want), name
    # layers 1..2 run three times: nine runs, each with a cache of its own; the input comes in again at runs 3 and 5
    spec = sepitar_model_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.pre_add_input for e in spec.schedule] == [False, False, False, True, False, True, False, False]
    assert all(e.cache is None for e in spec.schedule)
    assert [r[0] for r in SepitarConfig.from_dict(U.public(U.CONFIGS["odd"])).runs()] == [0, 1, 2, 0, 1, 2]
    assert [r[0] for r in P.layer_runs(U.CONFIGS["mix"])] == [e.layer for e in spec.schedule]
    for change, match in ((lambda c: c["layers"][0].__setitem__("type", "convolution"), "unknown mixer"),
                          (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "cannot be chosen"),
                          (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 18), "even and at most"),
                          (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "do not divide"),
                          (lambda c: c["loop"].__setitem__("stop", 9), "does not name a range"),
                          (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
                          (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank")):
        bad = copy.deepcopy(raw)
        change(bad)
        with pytest.raises(ConfigError, match=match):
            SepitarConfig.from_dict(bad)


def test_command_line_inspects_the_model(tmp_path):
    from zinfer_b200 import cli

    d = U.write_model(str(tmp_path / "m"), U.CONFIGS["mix"], U.make_weights(U.CONFIGS["mix"], seed=1))
    out = io.StringIO()
    assert cli.run(["inspect-config", d], out) == 0
    text = out.getvalue()
    assert "architecture: Sepitar" in text and "loop: layers 1..2 run 3 times" in text and "layer_runs: 8" in text
    assert "layer 1: attention (heads=4 kv_heads=2 dim=16 vdim=24 scale=0.6 bias_max=40 window=9)" in text
    assert "layer 2: attention_2 (heads=4 kv_heads=2 dim=16 vdim=8 scale=0.5 softcap=5.0 rot dims=8); feed-forward: none" in text
    assert "moe experts=4 top=3 ff=16 limit=0.8 shared ff=8 limit=1.0" in text
    out = io.StringIO()
    assert cli.run(["inspect-weights", d], out) == 0 and "tensor_count:" in out.getvalue()


def test_every_run_has_a_cache_of_its_own():
    from zinfer_b200.config import SepitarConfig, sepitar_model_spec
    from zinfer_b200.engine import DecoderModel

    model = DecoderModel(sepitar_model_spec(SepitarConfig.from_dict(U.public(U.CONFIGS["mix"]))), torch.float32, "cpu")
    kv, state = model.cache_needs()
    assert len(kv) == 8 and not state
    needs = [kv[r.cache] for r in model.runs]
    # latent attention: one row [latent | rotated key part] per token, keys only; its window is the layer's own
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].values, needs[0].window) == (1, 24, False, 11)
    assert needs[7].window == 5
    # the three runs of layer 1 (windows of 9) and of layer 2 (no window: every key stays)
    assert [n.window for n in needs[1:7]] == [9, None, 9, None, 9, None]
    assert (needs[1].num_kv_heads, needs[1].head_dim, needs[1].value_dim) == (2, 16, 24)
    assert (needs[2].num_kv_heads, needs[2].head_dim, needs[2].value_dim) == (2, 16, 8)


def test_weights_of_wrong_shape_are_refused(tmp_path):
    from zinfer_b200.engine import ModelRunner

    cfg = U.CONFIGS["odd"]
    w = U.make_weights(cfg, seed=2)
    w["l0.mix.g"] = torch.zeros(3, 44, dtype=torch.bfloat16)            # a gate per head where the layer has one per channel
    d = U.write_model(str(tmp_path / "bad"), cfg, w)
    with pytest.raises(Exception, match="l0.mix.g"):
        ModelRunner.from_model_dir(d, dtype=torch.float32, device="cpu", page_size=8, max_tokens=64, max_requests=2,
                                   cuda_graphs=False)
    w = U.make_weights(cfg, seed=2)
    del w["l1.mlp.router.b"]
    d = U.write_model(str(tmp_path / "less"), cfg, w)
    with pytest.raises(Exception, match="l1.mlp.router.b"):
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
    # the norm's weight is stored around zero
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    assert torch.allclose(P.norm_one_plus(x, torch.tensor([0.0, 1.0], dtype=F), 0.0), torch.tensor([[3.0, 8.0]], dtype=F) / 12.5 ** 0.5)
    # distance buckets of a table of 8 rows that ends at 64: one token per row up to 3, then steps of 64^(1/4)... = 2
    assert [P.distance_bucket(n, 8, 64.0) for n in (0, 1, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [0, 1, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    # rotation in halves: the second pair of four rotates by position * base^(-2/4)
    r = P.rotate_half(torch.tensor([[[0.0, 1.0, 0.0, 0.0, 9.0]]], dtype=F), torch.tensor([3]), [1.0, 0.25])
    assert torch.allclose(r, torch.tensor([[[0.0, np.cos(0.75), 0.0, np.sin(0.75), 9.0]]], dtype=F))
    # rotation of neighbours, with a magnitude: (1, 0) at position 2 with frequency 0.5 -> m (cos 1, sin 1); the rest passes
    r = P.rotate_pairs(torch.tensor([[[1.0, 0.0, 5.0]]], dtype=F), torch.tensor([2]), [0.5], magnitude=1.5)
    assert torch.allclose(r, torch.tensor([[[1.5 * np.cos(1.0), 1.5 * np.sin(1.0), 5.0]]], dtype=F))
    # frequencies by wavelength: short waves stay, long ones are divided, between them a blend
    rot = {"base": 100.0, "dims": 6, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    f = P.frequencies_by_wavelength(rot)          # wavelengths 6.28, 29.2, 135: below 16, between, above 64
    base = [1.0, 100.0 ** (-1 / 3), 100.0 ** (-2 / 3)]
    s = (64 / (2 * math.pi / base[1]) - 1.0) / 3.0
    assert np.allclose(f, [base[0], (1 - s) * base[1] / 4 + s * base[1], base[2] / 4])
    # the ramp: pairs below `lo` keep their frequency, pairs from `hi` on are divided by the factor
    rot = {"base": 10000.0, "dims": 8, "scaling": {"factor": 10.0, "original": 100, "fast": 8.0, "slow": 0.5}}
    f, mag = P.frequencies_ramped(rot)
    where = lambda t: 8 * math.log(100 / (2 * math.pi * t)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(0.5)), 7)
    assert (lo, hi) == (0, 2) and abs(mag - (0.1 * math.log(10.0) + 1.0)) < 1e-15
    plain = [10000.0 ** (-2 * i / 8) for i in range(4)]
    assert np.allclose(f, [plain[0], plain[1] * (0.5 / 10 + 0.5), plain[2] / 10, plain[3] / 10])
    # softmax with a sink: one key of score 0 and a sink of 0 share the weight; the sink has no value
    out = P.attend(torch.zeros(1, 1, 1, dtype=F), torch.tensor([[[2.0, 4.0]]], dtype=F), torch.ones(1, 1, dtype=torch.bool),
                   sink=torch.zeros(1, dtype=F))
    assert torch.allclose(out, torch.tensor([[1.0, 2.0]], dtype=F))
    # the window: position 6 with a window of 3 sees 4, 5, 6
    assert P.causal(torch.tensor([6]), 9, 3)[0].nonzero().flatten().tolist() == [4, 5, 6]
    # routing: the two largest logits, softmax over them alone; a tie goes to the earlier expert
    chosen, w = P.route(torch.tensor([0.0, 2.0, 2.0, 1.0], dtype=F), 2)
    assert chosen == [1, 2] and torch.allclose(w, torch.tensor([0.5, 0.5], dtype=F))
    chosen, w = P.route(torch.tensor([0.0, math.log(3.0), -5.0], dtype=F), 2)
    assert chosen == [1, 0] and torch.allclose(w, torch.tensor([0.75, 0.25], dtype=F))
    # the expert: gate 3 -> min(3, 2) = 2, up -5 -> -2: 2 sigmoid(3.404) (-2 + 1)
    one = torch.ones(1, 1, dtype=F)
    y = P.expert(one, torch.tensor([[3.0]], dtype=F), torch.tensor([[-5.0]], dtype=F), one, 2.0)
    assert abs(y.item() + 2.0 / (1.0 + math.exp(-3.404))) < 1e-12


def test_distance_buckets_of_the_engine_match_the_plain_ones():
    from zinfer_b200.parts.attention import distance_buckets

    for rows, far in ((4, 9.0), (8, 64.0), (12, 40.0), (32, 240.0), (6, 13.0), (16, 512.0)):
        got = distance_buckets(rows, far)
        assert got == [P.distance_bucket(n, rows, far) for n in range(len(got))]
        assert got[-1] == rows - 1 and P.distance_bucket(10 * len(got), rows, far) == rows - 1


def test_rescaled_frequencies_of_the_engine_match_the_plain_ones():
    from zinfer_b200.parts.rope import scaled_frequencies

    for cfg in U.CONFIGS.values():
        for lay in cfg["layers"]:
            rot = lay["mixer"].get("rot")
            if lay["type"] == "attention_2":
                f, mag = scaled_frequencies(rot["dims"], rot["base"], {"kind": "by_wavelength", **rot["scaling"]})
                assert np.allclose(f, P.frequencies_by_wavelength(rot), rtol=1e-14) and mag == 1.0
            elif lay["type"] == "latent_attention":
                f, mag = scaled_frequencies(rot["dims"], rot["base"], {"kind": "ramp", **rot["scaling"]})
                pf, pm = P.frequencies_ramped(rot)
                assert np.allclose(f, pf, rtol=1e-14) and abs(mag - pm) < 1e-15


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


# ---------------------------------------------------------------- edges of windows, sinks, distance tables, far keys
def _peaky(kind, mixer, rel_rows=None, width=64, vocab=149):
    """One layer of the given mixer without a feed-forward, whose output projection weighs as much as the embedding."""
    cfg = U.config(vocab, width, [U.layer(kind, mixer, None)], rel_rows={0: rel_rows} if rel_rows else None)
    w = U.make_weights(cfg, seed=31)
    w["l0.mix.o"] = (w["l0.mix.o"].float() * 4.0).to(torch.bfloat16)
    return cfg, w


EDGES = {
    # windows that end inside a page, at a page's edge and beyond several pages; scores peaky enough that one key more or
    # fewer at the window's edge moves the logits
    "attention": ("attention", U.att(4, 2, 16, 24, 1.2, 21, 60), 14),
    "attention_tensor_sizes": ("attention", U.att(4, 1, 64, 64, 0.5, 50, 100), 20),
    "latent": ("latent_attention", U.lat(3, 16, 8, 16, 24, 12, 0.9, 19), None),
    "latent_tensor_sizes": ("latent_attention", U.lat(4, 32, 32, 32, 96, 48, 0.35, 40), None),
}


def _wrong(cfg, weights, reqs):
    """The plain model's logits with a window one key wider or narrower, without the sink, and with the distance table
    read one row off: what an engine with that fault would give."""
    out = {}
    right_mask, right_bucket = P.causal, P.distance_bucket
    try:
        P.causal = lambda pos, n, window=None: right_mask(pos, n, None if window is None else window + 1)
        out["window one too wide"] = U.plain_logits(cfg, weights, reqs)
        P.causal = lambda pos, n, window=None: right_mask(pos, n, None if window is None else window - 1)
        out["window one too narrow"] = U.plain_logits(cfg, weights, reqs)
        P.causal = right_mask
        if cfg["layers"][0]["type"] == "attention":
            P.distance_bucket = lambda n, rows, far: right_bucket(max(n - 1, 0), rows, far)
            out["distance one off"] = U.plain_logits(cfg, weights, reqs)
            P.distance_bucket = right_bucket
        else:
            out["no sink"] = U.plain_logits(cfg, weights, reqs, sink=False)
    finally:
        P.causal, P.distance_bucket = right_mask, right_bucket
    return out


@pytest.mark.parametrize("case", ["attention", "latent"])
def test_the_peaky_requests_show_every_fault_of_the_mask(case):
    """The plain model alone: with a window one key wider or narrower, without the sink or with the distance table one
    row off, the logits move by more than the loosest tolerance of the tests below at many positions."""
    kind, mixer, rel = EDGES[case]
    cfg, weights = _peaky(kind, mixer, rel)
    reqs = ru.make_requests(cfg["vocab"], [90], seed=6)
    plain = U.plain_logits(cfg, weights, reqs)
    for what, other in _wrong(cfg, weights, reqs).items():
        moved = np.abs(other["r0"] - plain["r0"]).max(axis=-1) / np.abs(plain["r0"]).max(axis=-1)
        # (with scores this peaky the sink weighs little beyond the first tokens: it has a test of its own)
        assert (moved > 2 * TOL[torch.bfloat16]["rtol"]).sum() >= (1 if what == "no sink" else 5), (what, moved.max())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", list(EDGES))
def test_every_edge_of_the_window_decides(tmp_path, dtype, case):
    """Prompts of a few hundred tokens with peaky attention (the test above shows that each fault of the mask moves
    these logits by far more than the tolerance): whole, in portions that end around page edges and window edges,
    decoding token by token far past the window (so that pages leave it and are used again), and mixed."""
    kind, mixer, rel = EDGES[case]
    cfg, weights = _peaky(kind, mixer, rel)
    window = mixer["mask"]["size"]
    page = 16
    n = 3 * window + 70
    reqs = ru.make_requests(cfg["vocab"], [n, window + 2, window, 3], seed=6)
    plain = U.plain_logits(cfg, weights, reqs)
    runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=page, max_tokens=2 * (n + page) + 4 * page,
                         max_requests=3, poison_freed_pages=True)
    edges = (page, page - 1, 1, page + 1, 2 * page - 1, 2, window, 2, window - 1, 3, window + 1, 1, 1, 5, 40)
    for mode, trace in (("whole", ru.trace_whole(reqs)), ("edges", ru.trace_portions(reqs, 0, sizes=edges)),
                        ("long decode", ru.trace_tail_decode(reqs, 2 * window + 30)),
                        ("mixed", ru.trace_mixed(reqs, 3, max_live=3, tail=window + 9))):
        got = ru.run_in_process(runner, trace)
        ru.assert_close(got, plain, what=f"edges {case}/{mode}", argmax_frac=0.0, **TOL[dtype])
    assert runner.graphs is not None and runner.graphs.replays > window
    assert sum(g.pool.reused for g in runner.manager.groups) > 0
    runner.manager.check()


@gpu
@pytest.mark.parametrize("kind", ["attention_2", "latent_attention"])
def test_the_sink_carries_the_first_tokens(tmp_path, kind):
    """With small scores and large sinks the sink holds most of the softmax's denominator at a sequence's first tokens:
    the plain model without it gives other logits by far, and the engine matches the one with it."""
    for big in (False, True):
        d = 64 if big else 8
        mixer = U.att2(2, 1, d, d, 0.3 / d ** 0.5, 20.0, d // 2) if kind == "attention_2" else \
            U.lat(2, d, d // 2, d, 2 * d, d, 0.3 / d ** 0.5, 6)
        cfg, weights = _peaky(kind, mixer, width=32, vocab=61)
        weights["l0.mix.sink"] = torch.tensor([2.0, -1.0], dtype=torch.bfloat16)
        reqs = ru.make_requests(cfg["vocab"], [12, 2, 1], seed=9)
        plain = U.plain_logits(cfg, weights, reqs)
        no_sink = U.plain_logits(cfg, weights, reqs, sink=False)
        assert all(np.abs(plain[r] - no_sink[r]).max() > 0.1 * np.abs(plain[r]).max() for r in reqs)
        for dtype in (torch.float32, torch.bfloat16):
            runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
            for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 11), ru.trace_portions(reqs, 3, sizes=(2, 1, 2, 3))):
                ru.assert_close(ru.run_in_process(runner, trace), plain, what="sink", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_the_cap_on_the_scores_bites(tmp_path):
    """Scores several times the cap: without the cap the softmax would be one-hot, with it many keys share the weight."""
    mixer = U.att2(2, 1, 16, 16, 2.0, 1.5, 8)
    cfg, weights = _peaky("attention_2", mixer, width=32, vocab=61)
    reqs = ru.make_requests(cfg["vocab"], [40, 5], seed=3)
    plain = U.plain_logits(cfg, weights, reqs)
    loose = copy.deepcopy(cfg)
    loose["layers"][0]["mixer"]["softcap"] = 1e6
    other = U.plain_logits(loose, weights, reqs)
    assert np.abs(plain["r0"] - other["r0"]).max() > 0.2 * np.abs(plain["r0"]).max()
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
        for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 9)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="cap", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_a_single_far_key_decides(tmp_path):
    """One key hundreds of tokens back (the layer has no window) carries much of the last query's softmax: among all
    tokens that could stand at position 19, the test takes the one whose presence moves the last position's logits most
    in the plain model, and requires that move to be large; an engine that lost that key could not match."""
    cfg, weights = _peaky("attention_2", U.att2(2, 1, 8, 12, 1.5, 30.0, 4, base=100.0), width=32, vocab=67)
    toks = ru.make_requests(cfg["vocab"], [270], seed=7)["r0"]
    without = toks[:19] + [toks[18]] + toks[20:]
    lost = U.plain_logits(cfg, weights, {"r0": without})
    move = {c: np.abs(U.plain_logits(cfg, weights, {"r0": toks[:19] + [c] + toks[20:]})["r0"][-1] - lost["r0"][-1]).max()
            for c in range(0, cfg["vocab"], 3)}
    toks[19] = max(move, key=move.get)
    plain = U.plain_logits(cfg, weights, {"r0": toks})
    assert np.abs(plain["r0"][-1] - lost["r0"][-1]).max() > 0.05 * np.abs(plain["r0"][-1]).max()     # the far key matters
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=288, max_requests=1)
        for trace in (ru.trace_whole({"r0": toks}), ru.trace_tail_decode({"r0": toks}, 5)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="one far key", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_the_router_bias_changes_choices(tmp_path):
    """In the plain model the chosen experts differ with and without the router's bias; the engine matches the one with it."""
    cfg = U.MECHANISMS["experts"]
    weights = U.make_weights(cfg, seed=61)
    reqs = U.clear_requests(cfg, weights, [40, 7], seed=9, margin=0.05)
    plain = U.plain_logits(cfg, weights, reqs)
    zero = {**weights, "l0.mlp.router.b": torch.zeros_like(weights["l0.mlp.router.b"])}
    assert np.abs(U.plain_logits(cfg, zero, reqs)["r0"] - plain["r0"]).max() > 0.05 * np.abs(plain["r0"]).max()
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, max_tokens=64, max_requests=2)
        for trace in (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 9)):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what="router bias", argmax_frac=0.0, **TOL[dtype])


@gpu
def test_sizes_of_a_real_layer(tmp_path):
    """Heads of 64 and 128, a latent row of 192 values, rows the tensor-core products take: the fast kernels against the
    plain model, in prompts of a few hundred tokens, decoded tails and mixed batches."""
    cfg = U.config(257, 256, [
        U.layer("latent_attention", U.lat(4, 64, 32, 64, 160, 96, 0.1, 48), U.moe(128, 8, 2, 1.5, shared=(128, 2.0))),
        U.layer("attention", U.att(4, 2, 64, 64, 0.12, 40, 90), U.moe(128, 8, 2, 1.5)),
        U.layer("attention_2", U.att2(2, 1, 128, 128, 0.09, 20.0, 64), U.moe(64, 4, 1, 1.0, shared=(64, 1.0))),
    ], loop=(1, 3, 2), rel_rows={1: 16})
    weights = U.make_weights(cfg, seed=71)
    reqs = U.clear_requests(cfg, weights, [150, 37, 70, 5], seed=5, margin=0.05)
    plain = U.plain_logits(cfg, weights, reqs)
    for dtype in (torch.float32, torch.bfloat16):
        runner = make_runner(tmp_path, cfg, weights, dtype, DEV, page_size=16, max_tokens=400, max_requests=3, poison_freed_pages=True)
        for mode, trace in (("whole", ru.trace_whole(reqs)), ("tail", ru.trace_tail_decode(reqs, 60)),
                            ("portions", ru.trace_portions(reqs, 4, sizes=(33, 2, 64, 17, 1, 40))),
                            ("mixed", ru.trace_mixed(reqs, 2, max_live=3, tail=20))):
            ru.assert_close(ru.run_in_process(runner, trace), plain, what=f"real sizes/{mode}", argmax_frac=0.0, **TOL[dtype])
        runner.manager.check()
        if dtype == torch.bfloat16:
            # a prompt and a single token ran on the tensor-core kernels, not on the exact ones
            from zinfer_b200 import profiling
            from zinfer_b200.engine import StepEntry
            with profiling.profile() as prof:
                runner.step([StepEntry("p", reqs["r0"][:100], [99])])
                runner.step([StepEntry("p", reqs["r0"][100:101], [0])])
            runner.end_request("p")
            ran = {c["class"] for c in prof.summary()["classes"]}
            assert {"attention (prefill, mma.sync, changed scores)", "attention (decode, changed scores)",
                    "latent attention (decode, split keys)", "latent attention: causal softmax"} <= ran, ran
            assert not {"attention (exact, CUDA cores)", "latent attention (exact, CUDA cores)"} & ran, ran


@gpu
def test_fast_kernels_agree_with_the_exact_ones(tmp_path, monkeypatch):
    """The same bfloat16 model on the tensor-core attention kernels and on the exact kernels: whole prompts, portions
    and single tokens agree to the rounding of the softmax weights' second part."""
    from zinfer_b200 import ops

    cfg = U.config(131, 128, [
        U.layer("attention", U.att(8, 2, 64, 64, 0.25, 70, 200), None),
        U.layer("attention_2", U.att2(4, 4, 128, 128, 0.2, 8.0, 32), None),
        U.layer("latent_attention", U.lat(20, 16, 16, 16, 48, 24, 0.4, 45), None),      # more heads than one block of the decode kernel takes
    ], rel_rows={0: 24})
    weights = U.make_weights(cfg, seed=81)
    reqs = ru.make_requests(cfg["vocab"], [300, 130, 33], seed=2)
    traces = (ru.trace_whole(reqs), ru.trace_tail_decode(reqs, 20), ru.trace_portions(reqs, 5, sizes=(64, 3, 129, 32, 1, 40)),
              ru.trace_mixed(reqs, 4, max_live=3, tail=12))
    got = {}
    for backend in ("generic", "auto"):
        monkeypatch.setattr(ops, "ATTENTION_BACKEND", backend)
        runner = make_runner(tmp_path, cfg, weights, torch.bfloat16, DEV, page_size=16, max_tokens=640, max_requests=3)
        got[backend] = [ru.run_in_process(runner, t) for t in traces]
    for exact, fast in zip(got["generic"], got["auto"]):
        for key, row in exact.items():
            assert np.abs(fast[key] - row).max() <= 2e-2 * np.abs(row).max(), key


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
        assert len(r.token_ids) == 25                              # past the windows of 5, 9 and 11 tokens
        logits = P.Plain(cfg, weights).forward(p + r.token_ids).numpy()
        for i, t in enumerate(r.token_ids):      # the best token given the same history, or tied with it to rounding
            row = logits[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-4 * np.abs(row).max()


@gpu
def test_command_line_makes_a_random_model_and_generates(tmp_path):
    """bin/zinfer: a model folder of random weights made from a Sepitar config.json, then tokens from it, greedy and sampled."""
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(U.public(U.CONFIGS["odd"])))
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


# ------------------------------------------------------------------ the new kernels alone, against their plain stand-ins
@gpu
def test_row_kernels_against_plain_arithmetic():
    """zi_qkv_rows_prepare, zi_rmsnorm_rows, zi_latent_prepare_rows, zi_rope_table_freqs: each against a few lines of PyTorch,
    for 32-bit sources beside 16-bit results and for one type throughout, few rows (the wide form) and many."""
    import kernel_refs as R
    from zinfer_b200 import ops

    g = torch.Generator(device=DEV).manual_seed(5)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=DEV)
    freqs = torch.tensor([1.0, 0.31, 0.07, 0.002], device=DEV)
    cos, sin = ops.rope_table_freqs(300, freqs, 1.25)
    rc, rs = R.rope_table_freqs(300, freqs, 1.25)
    assert torch.allclose(cos, rc, atol=1e-6) and torch.allclose(sin, rs, atol=1e-6)
    for T, out_dtype in ((5, torch.bfloat16), (200, torch.bfloat16), (7, torch.float32)):
        nq, nkv, d, dv, n_gate, page, rot = 6, 2, 12, 20, 6, 8, 8
        width = nq * d + nkv * d + nkv * dv + n_gate
        proj = rnd(T, width)
        bias, qw, kw = rnd(width) * 0.3, 1 + 0.2 * rnd(nq * d), 1 + 0.2 * rnd(nkv * d)
        pos = torch.randint(0, 300, (T,), generator=g, device=DEV, dtype=torch.int32)
        slots = torch.randperm(40 * page, generator=g, device=DEV)[:T].to(torch.int32)
        slots[0] = -1                                                   # a row that pads a captured batch writes nothing
        caches = [[torch.zeros(40, nkv, page, n, dtype=out_dtype, device=DEV) for n in (d, dv)] for _ in range(2)]
        got = ops.qkv_rows_prepare(proj, bias, nq, nkv, d, dv, n_gate, qw, kw, 1e-5, rot, cos, sin, pos, *caches[0], slots, page, out_dtype)
        want = R.qkv_rows_prepare(proj, bias, nq, nkv, d, dv, n_gate, qw, kw, 1e-5, rot, cos, sin, pos, *caches[1], slots, page, out_dtype)
        tol = dict(rtol=2e-2, atol=2e-2) if out_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
        for a, b in zip((*got, *caches[0]), (*want, *caches[1])):
            assert torch.allclose(a.float(), b.float(), **tol)
        assert caches[0][0].abs().sum() > 0
        x = rnd(T, 50)[:, 3:40]                                         # a view of wider rows
        w = 1 + 0.2 * rnd(37)
        assert torch.allclose(ops.rmsnorm_rows(x, w, 1e-6, out_dtype).float(), R.rmsnorm_rows(x, w, 1e-6, out_dtype).float(), **tol)
        for neighbours in (False, True):
            heads, dim, rd, rank = 3, 10, 8, 14
            D = rank + rd
            q, kv, cw = rnd(T, heads * (dim + rd)).to(out_dtype), rnd(T, D + 5), 1 + 0.2 * rnd(rank)
            outs = []
            for fn in (ops.latent_prepare_rows, R.latent_prepare_rows):
                q_eff = torch.zeros(T, heads, D, dtype=out_dtype, device=DEV)
                cache = torch.zeros(40, 1, page, D, dtype=out_dtype, device=DEV)
                fn(q, kv, heads, dim, rd, rank, rd, neighbours, cw, 1e-5, cos, sin, pos, q_eff, cache, slots)
                outs.append((q_eff[:, :, rank:].float(), cache.float()))
            assert all(torch.allclose(a, b, **tol) for a, b in zip(*outs))


@gpu
def test_clamped_gate_grouped_gate_and_the_logits_router():
    import kernel_refs as R
    from zinfer_b200 import ops

    g = torch.Generator(device=DEV).manual_seed(6)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device=DEV)
    for T, I, dtype in ((3, 24, torch.bfloat16), (130, 64, torch.bfloat16), (9, 7, torch.float32), (40, 16, torch.float32)):
        gu = (3.0 * rnd(T, 2 * I)).to(dtype)
        tol = dict(rtol=2e-2, atol=1e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-6)
        got, want = ops.clamped_gate(gu, 1.5, 1.702, 1.0, dtype), R.clamped_gate(gu, 1.5, 1.702, 1.0, dtype)
        assert torch.allclose(got.float(), want.float(), **tol) and want.float().abs().max() > 1.0
        parts = ops.Partials(torch.stack([gu.float() * 0.25, gu.float() * 0.75]).contiguous())       # split-K partial sums, added in order
        assert torch.allclose(ops.clamped_gate(parts, 1.5, 1.702, 1.0, dtype).float(), want.float(), **tol)
        x, gate = rnd(T, 4 * I).to(dtype), rnd(T, 4).to(dtype)
        assert torch.allclose(ops.sigmoid_gate(x, gate, group=I).float(), R.sigmoid_gate(x, gate, group=I).float(), **tol)
    for T, K, NR, top in ((1, 64, 8, 4), (70, 192, 5, 5), (9, 33, 12, 1)):
        x, w, b = rnd(T, K).to(torch.bfloat16), rnd(NR, K).to(torch.bfloat16), rnd(NR)
        w[1] = w[0]                                                      # equal logits unless the bias parts them
        b[1] = b[0]                                                      # a tie: the earlier expert first
        chosen, weight = ops.moe_router_top_logits(x, w, b, top)
        rc, rw = R.moe_router_top_logits(x, w, b, top)
        z = x.float() @ w.float().T + b
        for t in range(T):
            # the same experts in the same order wherever the logits are clearly apart
            gaps = z[t].sort(descending=True).values
            clear = all(float(gaps[k] - gaps[k + 1]) > 1e-3 or float(gaps[k] - gaps[k + 1]) == 0.0 for k in range(min(top, NR - 1)))
            if clear:
                assert chosen[t].tolist() == rc[t].tolist(), (t, chosen[t], rc[t])
                assert torch.allclose(weight[t], rw[t], rtol=1e-4, atol=1e-6)
        assert torch.allclose(weight.sum(-1), torch.ones(T, device=DEV), atol=1e-5)
