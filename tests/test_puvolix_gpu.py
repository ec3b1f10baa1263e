"""Whole Puvolix models through the engine against the plain implementation: every cutting of the requests into
steps, both precisions, other orders of layers, long decoding, slots and pages that are used again, generation
through the scheduler and the command line."""

from __future__ import annotations

import json
import math

import pytest
import torch

from tests import helpers as H
from tests.plain import puvolix_plain as P

pytestmark = pytest.mark.gpu


def _left(heads, kv, dim, vdim, conv, rot=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale or dim ** -0.5}
    if rot is not None:
        dims, base, scaling = rot
        m["rot"] = {"dims": dims, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return m


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(left, right, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _config(vocab, width, layers, eps=1e-5, groups=1, softcap=0.0):
    return {"architecture": "Puvolix", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "logit_softcap": softcap, "layers": layers}


# Configurations that differ in every size and option: several kv heads and groups of recurrent heads, head sizes
# that are no multiples of 8 or of 16, key and value sizes that differ either way, convolutions of one to five taps,
# rotation of the whole head, of a part and none, frequency ladders that reach all three wavelength ranges, one to
# six norm groups, dense, routed (one to three chosen; with and without a shared expert) and no feed-forward, with
# and without a cap on the logits.
CONFIGS = {
    "A": _config(97, 48, [
        _layer(_left(4, 2, 12, 20, 2, (8, 100.0, (3.0, 1.0, 3.0, 40))), _right(4, 2, 12, 20, 3), _dense(40)),
        _layer(_left(6, 3, 8, 8, 4, (8, 5000.0, None)), _right(2, 1, 24, 8, 2), _moe(5, 2, 24, 1.2, (16, 0.8))),
        _layer(_left(2, 2, 20, 12, 1), _right(3, 3, 10, 14, 5), _moe(3, 1, 16, 2.5))], groups=3, softcap=8.0),
    "B": _config(130, 96, [
        _layer(_left(3, 1, 24, 40, 5, (24, 30.0, (8.0, 0.5, 2.0, 64))), _right(6, 2, 16, 12, 1), None),
        _layer(_left(8, 4, 12, 12, 3, (4, 1e4, None)), _right(2, 2, 40, 24, 4), _moe(4, 3, 32, 0.7, (8, 3.0))),
        _layer(_left(2, 1, 36, 6, 2, (36, 250.0, (2.0, 1.0, 8.0, 16))), _right(4, 1, 24, 20, 3), _dense(72)),
        _layer(_left(4, 4, 16, 16, 3, (16, 77.0, None)), _right(1, 1, 32, 32, 2), _moe(2, 2, 48, 1.0))], eps=1e-6, groups=1),
    "C": _config(61, 44, [
        _layer(_left(2, 1, 22, 10, 3, (10, 9.0, (4.0, 1.0, 4.0, 30))), _right(2, 1, 18, 26, 2), _moe(9, 1, 8, 1.5, (12, 1.0))),
        _layer(_left(1, 1, 44, 44, 2, (44, 1e5, None)), _right(4, 4, 6, 6, 4), None)], eps=1e-4, groups=4, softcap=30.0),
    # shapes that the tensor-core kernels take in bfloat16: widths and expert sizes that are multiples of 8, key
    # and value sizes that are multiples of 16 (equal and unequal)
    "D": _config(111, 128, [
        _layer(_left(4, 2, 64, 64, 3, (32, 1e4, (4.0, 1.0, 4.0, 128))), _right(4, 2, 32, 32, 4), _moe(8, 2, 32, 1.5, (64, 1.0))),
        _layer(_left(8, 2, 48, 32, 2, (32, 1e5, (8.0, 1.0, 4.0, 512))), _right(4, 2, 64, 32, 3), _dense(96)),
        _layer(_left(2, 2, 128, 64, 2, (64, 500.0, None)), _right(2, 1, 64, 64, 2), _moe(4, 1, 64, 2.0))], groups=4, softcap=20.0),
    # no routed layer: in bfloat16 every position of every request is compared (no choice that rounding could turn)
    "E": _config(83, 64, [
        _layer(_left(4, 2, 16, 24, 3, (8, 1000.0, (2.0, 1.0, 2.0, 20))), _right(4, 2, 16, 8, 4), _dense(48)),
        _layer(_left(2, 1, 32, 32, 4, (32, 50.0, None)), _right(2, 2, 24, 16, 3), None),
        _layer(_left(4, 4, 8, 12, 2), _right(8, 2, 8, 8, 2), _dense(32))], groups=2, softcap=12.0),
}


def _folder(tmp_path_factory, name, cfg=None, seed=None):
    from quanta_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    d = tmp_path_factory.mktemp(f"puvolix_{name}")
    weights = P.draw_weights(cfg, seed=(500 + ord(name[0])) if seed is None else seed)
    write_safetensors(d / "model.safetensors", weights)
    (d / "config.json").write_text(json.dumps(cfg))
    return d, weights, cfg


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: _folder(tmp_path_factory, name) for name in CONFIGS}


def _engine(folder, dtype, steps=None, page_size=16, slots=4, num_pages=None):
    from quanta_b200.engine.model import load_model
    from quanta_b200.engine.step import Engine
    model, _ = load_model(folder, dtype=dtype)
    if num_pages is None:
        num_pages = H.tokens_in_flight(steps, page_size) // page_size
    return Engine(model, num_pages=num_pages, page_size=page_size, max_requests=slots)


def _want(weights, cfg, reqs):
    """Logits of every position and, per position, the smallest routing margin of any layer at this position or an
    earlier one of the request."""
    out, margin = {}, {}
    for rid, toks in reqs.items():
        lg, info = P.forward(weights, cfg, toks, details=True)
        routing = info["routing"]
        m = torch.stack([mg for _, mg in routing]).min(0).values if routing else torch.full((len(toks),), 1e9)
        m = torch.cummin(m, 0).values
        for i in range(len(toks)):
            out[(rid, i)] = lg[i]
            margin[(rid, i)] = float(m[i])
    return out, margin


def _replay_following_the_routing(eng, steps, weights, cfg, reqs):
    """Replay ``steps`` while the routed layers report what every token chose; then the plain implementation's logits
    with those choices forced.  In bfloat16 a close choice may turn, and everything above it then differs for a reason
    that is no fault; following the engine's choices compares everything else at every position."""
    from quanta_b200.engine.step import StepEntry
    routed = [eng.model.blocks[e.layer].feed_forward for e in eng.model.schedule
              if hasattr(eng.model.blocks[e.layer].feed_forward, "trace")]
    for part in routed:
        part.trace = []
    eng.use_graphs = False
    got, chosen, pos = {}, {rid: [[None] * len(t) for _ in routed] for rid, t in reqs.items()}, {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], tuple(e["want"])) for e in s["entries"]]
        logits = eng.step(entries, end=s["end"])
        eng.check()
        logits = logits.float().cpu() if logits is not None else None
        picks = [part.trace.pop(0).cpu() for part in routed]
        row = lrow = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = logits[lrow]
                lrow += 1
            for i in range(len(e["tokens"])):
                for l in range(len(routed)):
                    chosen[e["id"]][l][base + i] = picks[l][row].tolist()
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    want, shake = {}, {}
    noisy = dict(weights)
    g = torch.Generator().manual_seed(1)
    noisy["embed"] = (weights["embed"].float() * (1 + 2.0 ** -8 * torch.randn(weights["embed"].shape, generator=g)))
    for rid, toks in reqs.items():
        picks = [torch.tensor(c) for c in chosen[rid]]
        lg = P.forward(weights, cfg, toks, chosen=picks)
        # where the model itself turns a rounding of its input into a large difference (a per-head norm of a state
        # that is nearly zero after the first tokens, a softmax between two nearly equal large scores), bfloat16
        # results say nothing about the engine: the plain model with its input disturbed by 2^-8 shows where
        shaken = P.forward(noisy, cfg, toks, chosen=picks)
        for i in range(len(toks)):
            want[(rid, i)] = lg[i]
            d = shaken[i] - lg[i]
            shake[(rid, i)] = float((d - d.mean()).pow(2).mean().sqrt() / lg[i].std())
    return got, want, shake


def _errors(got, want):
    err = {}
    for key, row in got.items():
        ref = want[key]
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / ref.std())
        err[key] = e if e == e else math.inf
    return err


def _worst(got, want, margins=None, near_tie=0.0, shake=None):
    """Largest error and where.  ``margins``: positions after a close routing choice are left out.  ``shake``: what
    the plain model makes of a small disturbance of its input, per position; the error is counted beyond six times
    that (bfloat16 rounds at every sublayer), and most positions must be steady enough for the test to say something."""
    err = _errors(got, want)
    if shake is not None:
        assert sum(1 for k in err if 6 * shake[k] < 0.2) >= 0.6 * len(err), "the model is unsteady nearly everywhere"
        err = {k: max(0.0, e - 6 * shake[k]) for k, e in err.items()}
    keys = [k for k in err if margins is None or margins[k] >= near_tie]
    assert len(keys) >= 0.25 * len(err), "too many positions after a close routing choice: the test would show nothing"
    where = max(keys, key=lambda k: err[k])
    return err[where], where


TOL = {"float32": 2e-4, "bfloat16": 0.1}
NEAR_TIE = {"float32": 1e-5}


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


def _compare(folder, weights, cfg, reqs, steps, dtype, what, **engine_args):
    eng = _engine(folder, dtype, steps, **engine_args)
    if dtype == "bfloat16":
        got, following, shake = _replay_following_the_routing(eng, steps, weights, cfg, reqs)
        worst, where = _worst(got, following, shake=shake)
    else:
        want, margins = _want(weights, cfg, reqs)
        got = H.replay(eng, steps)
        worst, where = _worst(got, want, margins, NEAR_TIE[dtype])
    assert len(got) == sum(len(t) for t in reqs.values())
    assert worst < TOL[dtype], f"{what} {dtype}: {worst} at {where}"
    eng.manager.check_invariants()
    assert eng.manager.stats()["live_requests"] == 0
    return eng


# ---- whole models under every cutting ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_cuttings_agree_with_plain(models, name, dtype):
    folder, weights, cfg = models[name]
    reqs = _requests(cfg["vocab"], [1, 2, 37, 70, 5, 110], seed=11)
    cuttings = {
        "whole": H.cut_whole(reqs),
        "decode": H.cut_tail_decode(reqs, tail=45),
        "portions": H.cut_portions(reqs, sizes=(7, 2, 13, 3, 1, 2, 29, 4, 16, 2)),
        "mixed": H.cut_mixed(reqs, max_live=3, seed=5, portion_sizes=(2, 3, 5, 8, 17, 33)),
    }
    for cut, steps in cuttings.items():
        # exactly the pages the cutting needs and three state slots: both are given back and used again
        _compare(folder, weights, cfg, reqs, steps, dtype, f"{name} {cut}", page_size=8 if name in "ACE" else 16, slots=3)


_FF = _moe(4, 2, 16, 1.3, (8, 0.9))
ORDERS = {
    # one layer only (the weighted sum has two terms), layers without any feed-forward, dense only, routed only,
    # a dense layer between routed ones, layers whose two branches differ from layer to layer
    "one_layer": [_layer(_left(2, 1, 16, 8, 3, (16, 30.0, None)), _right(2, 1, 16, 8, 2), _FF)],
    "mixers_only": [_layer(_left(2, 2, 8, 8, 2, (8, 100.0, None)), _right(2, 2, 8, 12, 3)),
                    _layer(_left(4, 1, 12, 8, 3), _right(4, 2, 8, 8, 4))],
    "dense_only": [_layer(_left(2, 1, 16, 16, 2, (8, 100.0, None)), _right(2, 1, 16, 16, 2), _dense(24)),
                   _layer(_left(2, 1, 16, 16, 2, (8, 100.0, None)), _right(2, 1, 16, 16, 2), _dense(56))],
    "routed_only": [_layer(_left(2, 1, 16, 16, 3, (16, 1e3, (4.0, 1.0, 4.0, 32))), _right(2, 2, 16, 16, 4), _FF),
                    _layer(_left(2, 1, 16, 16, 3, (16, 1e3, (4.0, 1.0, 4.0, 32))), _right(2, 2, 16, 16, 4), _moe(6, 3, 8, 0.5))],
    "dense_between": [_layer(_left(4, 2, 8, 12, 4, (4, 20.0, None)), _right(2, 1, 12, 8, 2), _FF),
                      _layer(_left(2, 1, 20, 8, 2, (20, 2e4, (16.0, 1.0, 2.0, 24))), _right(4, 4, 16, 8, 3), _dense(40)),
                      _layer(_left(1, 1, 24, 24, 3), _right(1, 1, 24, 24, 4), None),
                      _layer(_left(4, 2, 8, 12, 4, (4, 20.0, None)), _right(2, 1, 12, 8, 2), _FF)],
}


@pytest.mark.parametrize("order", list(ORDERS))
def test_other_orders_of_layers(tmp_path_factory, order):
    cfg = _config(67, 40, ORDERS[order], groups=2 if order != "one_layer" else 5, softcap=0.0 if order == "dense_only" else 15.0)
    folder, weights, cfg = _folder(tmp_path_factory, "A", cfg=cfg, seed=3)
    reqs = _requests(cfg["vocab"], [1, 40, 75], seed=1)
    steps = H.cut_mixed(reqs, max_live=3, seed=5, portion_sizes=(2, 3, 5, 8, 17))
    for dtype in ("float32", "bfloat16"):
        _compare(folder, weights, cfg, reqs, steps, dtype, order, slots=3)


def test_residual_stream_after_every_layer(models):
    """The stream that goes on after each layer (the model's own trace) against the plain implementation's."""
    from quanta_b200.engine.step import StepEntry
    for name in ("A", "C"):
        folder, weights, cfg = models[name]
        toks = H.random_tokens(29, cfg["vocab"], 3)
        _, info = P.forward(weights, cfg, toks, details=True)
        eng = _engine(folder, "float32", num_pages=8)
        eng.model.residual_trace = []
        eng.step([StepEntry("a", toks, (0,))], end=["a"])
        assert len(eng.model.residual_trace) == len(cfg["layers"])
        for i, got in enumerate(eng.model.residual_trace):
            want = info["layers"][i]
            assert torch.allclose(got.cpu(), want, atol=2e-4 * float(want.abs().max()), rtol=1e-4), (name, i)


def test_token_by_token_equals_whole_prompt(models):
    """Every token alone (the recurrence's state and both convolutions' inputs cross a step at every token) against
    the prompt in one step."""
    for name in ("A", "C"):
        folder, weights, cfg = models[name]
        reqs = _requests(cfg["vocab"], [45], seed=3)
        one = H.cut_tail_decode(reqs, tail=1000)
        whole = H.cut_whole(reqs)
        a = H.replay(_engine(folder, "float32", one, page_size=4), one)
        b = H.replay(_engine(folder, "float32", whole, page_size=4), whole)
        worst, where = _worst(a, b)
        assert worst < 2e-5, (name, worst, where)


def test_portions_of_two_tokens(models):
    """Portions shorter than the convolutions' reach (two tokens, one token) against the whole prompt."""
    folder, weights, cfg = models["B"]          # convolutions of up to five taps
    reqs = _requests(cfg["vocab"], [31], seed=8)
    steps = H.cut_portions(reqs, sizes=(2, 2, 1, 2, 3, 2, 1, 1, 2))
    want, margins = _want(weights, cfg, reqs)
    got = H.replay(_engine(folder, "float32", steps, page_size=4), steps)
    worst, where = _worst(got, want, margins, NEAR_TIE["float32"])
    assert worst < TOL["float32"], (worst, where)


def test_batch_does_not_change_a_request(models):
    """Unequal requests in one batch against each alone, float32: the same numbers to rounding."""
    folder, weights, cfg = models["D"]
    reqs = _requests(cfg["vocab"], [33, 3, 90, 64], seed=21)
    together = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()], "end": list(reqs)}]
    alone = H.cut_whole(reqs)
    a = H.replay(_engine(folder, "float32", together), together)
    b = H.replay(_engine(folder, "float32", alone), alone)
    worst, where = _worst(a, b)
    assert worst < 2e-5, (worst, where)


def test_long_decoding_through_captured_steps(models):
    """A short prompt and 150 single tokens (captured decode steps once the shape has been seen), for two requests
    side by side that cross page borders at different steps."""
    folder, weights, cfg = models["E"]
    reqs = _requests(cfg["vocab"], [157, 171], seed=4)
    steps = [{"entries": [{"id": "r0", "tokens": reqs["r0"][:7], "want": [6]}, {"id": "r1", "tokens": reqs["r1"][:21], "want": [20]}],
              "end": []}]
    for i in range(150):
        steps.append({"entries": [{"id": "r0", "tokens": [reqs["r0"][7 + i]], "want": [0]},
                                  {"id": "r1", "tokens": [reqs["r1"][21 + i]], "want": [0]}], "end": []})
    want, _ = _want(weights, cfg, reqs)
    for dtype in ("float32", "bfloat16"):
        eng = _engine(folder, dtype, num_pages=44, page_size=8)
        got = H.replay(eng, steps)
        assert eng.stats()["graph_replays"] > 100
        worst, where = _worst(got, {k: want[k] for k in got})
        assert worst < TOL[dtype], (dtype, worst, where)


def test_slots_and_pages_are_used_again(models):
    """One slot and the pages of one request: five requests one after the other, each starting from a zero state and
    empty convolution inputs although the slot and the pages still hold the last request's numbers."""
    folder, weights, cfg = models["A"]
    reqs = _requests(cfg["vocab"], [30, 30, 29, 31, 30], seed=9)
    steps = H.cut_portions(reqs, sizes=(9, 1, 20, 1))
    eng = _engine(folder, "float32", num_pages=8, page_size=4, slots=1)
    got = H.replay(eng, steps)
    want, margins = _want(weights, cfg, reqs)
    worst, where = _worst(got, want, margins, NEAR_TIE["float32"])
    assert worst < TOL["float32"], (worst, where)


def test_every_constant_counts(tmp_path_factory):
    """The engine agrees with the plain implementation on a model whose constants are all far from neutral, and a
    plain model with ONE constant or tensor changed is far off: none of them is a detail that this test could not
    see."""
    layers = [_layer(_left(4, 2, 16, 8, 3, (12, 40.0, (4.0, 1.0, 4.0, 24)), scale=0.4), _right(4, 2, 12, 10, 3), _dense(24)),
              _layer(_left(2, 1, 16, 16, 2, (16, 300.0, (2.0, 1.0, 2.0, 16)), scale=0.3), _right(2, 1, 16, 8, 4),
                     _moe(4, 2, 16, 0.8, (8, 0.6)))]
    cfg = _config(50, 48, layers, groups=3, softcap=6.0)
    folder, weights, cfg = _folder(tmp_path_factory, "A", cfg=cfg, seed=77)
    reqs = _requests(cfg["vocab"], [41], seed=2)
    steps = H.cut_portions(reqs, sizes=(2, 3, 1, 2, 4, 6, 1, 1, 1, 5, 3, 12))
    got = H.replay(_engine(folder, "float32", steps, page_size=4), steps)
    want, margins = _want(weights, cfg, reqs)
    worst, where = _worst(got, want, margins, NEAR_TIE["float32"])
    assert worst < TOL["float32"], (worst, where)

    def other(edit, w=None):
        c = json.loads(json.dumps(cfg))
        if edit is not None:
            edit(c)
        far, _ = _worst(got, _want(w or weights, c, reqs)[0])
        return far

    def setter(layer, path, value):
        def edit(c):
            m = c["layers"][layer]
            for key in path[:-1]:
                m = m[key]
            m[path[-1]] = value
        return edit

    def top(c, key, value):
        c[key] = value

    ones = lambda name: dict(weights, **{name: torch.ones_like(weights[name])})  # noqa: E731
    zeros = lambda name: dict(weights, **{name: torch.zeros_like(weights[name])})  # noqa: E731
    first_only = dict(weights)
    for n in ("l1.mix.left.q.conv", "l1.mix.left.k.conv", "l1.mix.left.v.conv"):
        t = torch.zeros_like(weights[n])
        t[:, -1] = weights[n][:, -1]
        first_only[n] = t
    newest_only = dict(weights, **{"l1.dwa": torch.tensor([0.0, 0.0, 1.0]).to(torch.bfloat16)})
    changed = {
        "scale": other(setter(0, ("mixer", "left", "scale"), 0.8)),
        "rotation base": other(setter(0, ("mixer", "left", "rot", "base"), 4.0)),
        "rotated part": other(setter(0, ("mixer", "left", "rot", "dims"), 4)),
        "no frequency scaling": other(lambda c: c["layers"][0]["mixer"]["left"]["rot"].pop("scaling")),
        "scaling factor": other(setter(1, ("mixer", "left", "rot", "scaling", "factor"), 8.0)),
        "scaling original": other(setter(1, ("mixer", "left", "rot", "scaling", "original"), 64)),
        "norm groups": other(lambda c: top(c["norm"], "groups", 1)),
        "eps": other(lambda c: top(c["norm"], "eps", 0.5)),
        "cap": other(lambda c: top(c, "logit_softcap", 0.0)),
        "expert limit": other(setter(1, ("mlp", "expert", "limit"), 8.0)),
        "shared limit": other(setter(1, ("mlp", "shared", "limit"), 8.0)),
        "no shared expert": other(setter(1, ("mlp", "shared"), None)),
        "one expert fewer chosen": other(setter(1, ("mlp", "router", "top"), 1)),
        "head temperatures": other(None, ones("l0.mix.left.temp")),
        "left convolution": other(None, first_only),
        "depth weights": other(None, newest_only),
        "branch gain": other(None, ones("l0.mix.right.out")),
        "q norm gain": other(None, ones("l1.mix.left.q.norm")),
        "dense biases": other(None, zeros("l0.mlp.gate.b")),
        "down bias": other(None, zeros("l0.mlp.down.b")),
        "decay bias": other(None, zeros("l0.mix.right.dt_bias")),
        "decay rate": other(None, zeros("l1.mix.right.A_log")),
        "per-head gain": other(None, ones("l1.mix.right.norm")),
    }
    for what, far in changed.items():
        assert far > 30 * TOL["float32"], (what, far)


def test_greedy_generation_through_the_scheduler(models):
    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    folder, weights, cfg = models["E"]
    prompts = [H.random_tokens(n, cfg["vocab"], 40 + n) for n in (9, 23, 4)]
    llm = LLM(str(folder), dtype="float32", page_size=4, num_pages=40, max_requests=2, max_step_tokens=16, prefill_chunk=6)
    got = generate(llm, prompts, max_new_tokens=12, eos_id=[])
    for p, g in zip(prompts, got):
        assert g == P.generate(weights, cfg, p, 12)
    assert llm.last_stats["cache"]["live_requests"] == 0


def test_command_line_and_random_weights(tmp_path):
    """``python -m quanta_b200 random-weights`` writes a folder for this architecture and ``generate`` runs it."""
    import subprocess
    import sys
    cfg = CONFIGS["C"]
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    out = tmp_path / "model"
    root = str(H.__file__).rsplit("/tests/", 1)[0]
    subprocess.run([sys.executable, "-m", "quanta_b200", "random-weights", "--config", str(tmp_path / "c.json"), "--seed", "3",
                    "--out", str(out)], check=True, cwd=root)
    r = subprocess.run([sys.executable, "-m", "quanta_b200", "generate", "--model", str(out), "--prompt-ids", "1,2,3,4,5",
                        "--max-new-tokens", "5", "--dtype", "float32", "--eos-id", "60"], check=True, capture_output=True,
                       text=True, cwd=root)
    ids = [int(x) for x in r.stdout.strip().split(",")]
    from safetensors.torch import load_file
    weights = load_file(str(out / "model.safetensors"))
    want = P.generate(weights, json.loads((out / "config.json").read_text()), [1, 2, 3, 4, 5], 5)
    if 60 in want:
        want = want[: want.index(60)]
    assert ids == want


def test_trace_program_replays_a_schedule(models, tmp_path):
    """The trace program on a mixed schedule of this architecture: the logits files against the plain implementation."""
    import subprocess
    import sys
    import numpy as np
    folder, weights, cfg = models["E"]
    reqs = _requests(cfg["vocab"], [40, 9, 66], seed=31)
    steps = H.cut_mixed(reqs, max_live=3, seed=2, portion_sizes=(2, 5, 17))
    lines = "".join(json.dumps({"step": n, "entries": s["entries"], "end": s["end"]}) + "\n" for n, s in enumerate(steps))
    root = str(H.__file__).rsplit("/tests/", 1)[0]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, root + "/bin/trace_run", "--model", str(folder), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", str(H.tokens_in_flight(steps))], input=lines, capture_output=True, text=True, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(steps))]
    want, _ = _want(weights, cfg, reqs)
    got, pos = {}, {}
    for n, s in enumerate(steps):
        rows = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        row = 0
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], base + w)] = torch.from_numpy(rows[row].copy())
                row += 1
            pos[e["id"]] = base + len(e["tokens"])
    assert len(got) == sum(len(t) for t in reqs.values())
    worst, where = _worst(got, want)
    assert worst < TOL["float32"], (worst, where)
