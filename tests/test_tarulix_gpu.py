"""The Tarulix decoder in the engine against the plain implementation (tests/plain/tarulix_plain.py).

Small configurations of the tests' own, weights drawn at a scale where every mechanism matters (distance biases and
sinks as large as the scores' spread, blending fractions away from 0 and 1, head mixing away from the identity,
decays over a wide range), and inputs made so that a fault shows where random numbers would hide it (one key that
outweighs all others just inside and just outside a window, a pooled block that is just seen, a state that must
survive hundreds of tokens and a portion of one token).
"""

import json
import math
import random

import pytest
import torch

from tests import helpers as H
from tests.plain import tarulix_plain as P

pytestmark = pytest.mark.gpu


def _attn(heads, kv_heads, dim, vdim, window, far, rows, v_mix=True, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim),
         "mask": {"size": window}, "bias_max": far, "bias_rows": rows, "v_mix": v_mix}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _par(heads, kv_heads, dim, vdim, window, pool, rot, cap, inner, state, rank, taps, weights=(0.75, 1.1), mlp=None, scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim),
            "mask": {"size": window, "pool": pool}, "softcap": cap}
    if rot is not None:
        left["rot"] = {"dims": rot[0], "base": rot[1]}
    right = {"inner": inner, "state": state, "dt_rank": rank, "conv": taps}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": weights[0], "right_scale": weights[1]},
            "mlp": mlp}


def _moe(experts, identity, top, ff, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    m["shared"] = None if not shared else {"ff": shared}
    return m


def _config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Tarulix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}


# Sizes that are no powers of two and differ from one another; they cover: key sizes unlike value sizes and head
# sizes that are no multiple of 8 (the element-by-element paths); one kv head for all query heads and as many as
# query heads; windows of 1 (the token alone), of a few tokens, and longer than any request; bias tables of 2 to 16
# rows with ladders that end inside and beyond the window; blending chains that start at layer 0 and later, and
# layers outside the chain; pooled blocks of 1, 3, 4 and 7 tokens, a layer without pooled blocks, rotation of a part
# of the head, of all of it and none, with and without a score cap; scans with states of 1 to 24 numbers a channel,
# 1 to 4 taps; routers with and without pass-through experts and shared experts, top 1, top 2 and every expert
# chosen; layers without a feed-forward; widths that are no multiple of 8.
CONFIGS = {
    "A": _config(97, 64, [
        _attn(4, 2, 16, 24, 9, 50, 8, mlp=_moe(5, 2, 2, 24, 16)),
        _par(4, 2, 24, 16, 11, 4, (8, 10000.0), 5.0, 48, 8, 4, 4, (0.7, 1.2), mlp=_moe(6, 1, 2, 24, 24)),
        _attn(4, 2, 16, 24, 17, 30, 12),
        _par(2, 1, 16, 40, 5, 3, (16, 500.0), 0.0, 40, 5, 3, 2, (1.1, 0.5), mlp=_moe(3, 0, 1, 16, 0))]),
    "B": _config(130, 96, [
        _attn(3, 3, 20, 12, 1, 40, 4, v_mix=False, mlp=_moe(4, 3, 3, 32, 8)),
        _attn(6, 1, 16, 16, 400, 600, 16, mlp=_moe(2, 2, 4, 16, 32)),
        _par(6, 3, 12, 20, 7, 1, None, 2.0, 56, 1, 2, 1, mlp=None),
        _attn(6, 1, 16, 16, 6, 9, 6),
        _attn(2, 2, 40, 8, 23, 24, 2, v_mix=False, mlp=_moe(1, 1, 1, 8, 0))], eps=1e-6),
    "C": _config(61, 44, [
        _par(3, 3, 12, 20, 13, 7, (4, 100.0), 25.0, 20, 24, 5, 3, (0.5, 1.5), mlp=_moe(9, 4, 4, 8, 12)),
        _par(2, 1, 20, 12, 300, 4, (20, 2e5), 0.0, 36, 3, 1, 4, (1.0, 1.0)),
        _attn(1, 1, 24, 24, 31, 100, 10, mlp=_moe(3, 1, 2, 16, 0))], eps=1e-4),
    # shapes that the tensor-core products take in bfloat16: widths and expert sizes that are multiples of 8, heads
    # of 64 and 128
    "D": _config(111, 128, [
        _attn(4, 2, 64, 64, 33, 64, 12, mlp=_moe(8, 2, 2, 32, 64)),
        _par(4, 2, 64, 128, 20, 8, (32, 10000.0), 10.0, 128, 16, 8, 4, mlp=_moe(8, 0, 2, 64, 32)),
        _attn(4, 2, 64, 64, 50, 200, 8, mlp=_moe(4, 4, 2, 16, 16)),
        _par(2, 1, 128, 64, 16, 5, (64, 1e4), 0.0, 64, 8, 4, 2)]),
    # no routed layer: in bfloat16 every position of every request is compared (no choice that rounding could turn)
    "E": _config(83, 64, [
        _attn(4, 2, 32, 32, 10, 20, 8), _par(4, 4, 16, 24, 9, 4, (8, 1000.0), 8.0, 32, 6, 4, 3),
        _attn(4, 2, 32, 32, 21, 90, 14), _par(2, 1, 8, 12, 12, 6, (8, 50.0), 0.0, 24, 10, 2, 2, (1.3, 0.6))]),
}


def _file_config(cfg):
    """The configuration as a model folder holds it: the rows of a bias table are no key of the file."""
    cfg = json.loads(json.dumps(cfg))
    for layer in cfg["layers"]:
        layer["mixer"].pop("bias_rows", None)
    return cfg


def _folder(tmp_path_factory, name, cfg=None, seed=None):
    from quanta_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    d = tmp_path_factory.mktemp(f"tarulix_{name}")
    weights = P.draw_weights(cfg, seed=(300 + ord(name[0])) if seed is None else seed)
    write_safetensors(d / "model.safetensors", weights)
    (d / "config.json").write_text(json.dumps(_file_config(cfg)))
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
    earlier one of the request (a choice that rounding turns changes what the layers above keep of that token, and
    with it every later position)."""
    out, margin = {}, {}
    for rid, toks in reqs.items():
        lg, routing = P.forward(weights, cfg, toks, want_routing=True)
        m = torch.stack([mg for _, mg in routing]).min(0).values if routing else torch.full((len(toks),), 1e9)
        m = torch.cummin(m, 0).values
        for i in range(len(toks)):
            out[(rid, i)] = lg[i]
            margin[(rid, i)] = float(m[i])
    return out, margin


def _replay_following_the_routing(eng, steps, weights, cfg, reqs):
    """Replay ``steps`` while the routed layers report what every token chose; then the plain implementation's
    logits with those choices forced.  In bfloat16 a close choice may turn, and everything above it then differs
    for a reason that is no fault; following the engine's choices compares everything else (the weights of the
    chosen experts included) at every position."""
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
    want = {}
    for rid, toks in reqs.items():
        lg = P.forward(weights, cfg, toks, chosen=[torch.tensor(c) for c in chosen[rid]])
        for i in range(len(toks)):
            want[(rid, i)] = lg[i]
    return got, want


def _errors(got, want):
    err = {}
    for key, row in got.items():
        ref = want[key]
        d = row - ref
        e = float((d - d.mean()).pow(2).mean().sqrt() / ref.std())
        err[key] = e if e == e else math.inf
    return err


def _worst(got, want, margins=None, near_tie=0.0):
    """Largest difference of a row's logits (mean taken off) over the row's spread, and where; positions whose
    router margin is below ``near_tie`` (a choice that rounding may turn) are left out."""
    err = _errors(got, want)
    keys = [k for k in err if margins is None or margins[k] >= near_tie]
    assert len(keys) >= 0.25 * len(err), "too many positions after a close routing choice: the test would show nothing"
    where = max(keys, key=lambda k: err[k])
    return err[where], where


TOL = {"float32": 2e-4, "bfloat16": 0.12}
NEAR_TIE = {"float32": 1e-5}


def _requests(vocab, lengths, seed):
    return {f"r{i}": H.random_tokens(n, vocab, seed + i) for i, n in enumerate(lengths)}


def _compare(folder, weights, cfg, reqs, steps, dtype, what, **engine_args):
    eng = _engine(folder, dtype, steps, **engine_args)
    if dtype == "bfloat16":
        got, following = _replay_following_the_routing(eng, steps, weights, cfg, reqs)
        worst, where = _worst(got, following)
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


_FF = _moe(4, 1, 2, 16, 8)
ORDERS = {
    # no layer keeps a state (the engine has no slot arrays), none keeps a bias table or a sink, one layer only, a
    # blending chain of one layer (it blends nothing), three layers of a chain in a row, the two kinds in turn
    # starting with the parallel one
    "attention_only": [_attn(4, 2, 16, 16, 8, 20, 6, mlp=_FF), _attn(4, 2, 16, 16, 5, 20, 6, v_mix=False), _attn(4, 2, 16, 16, 12, 40, 10)],
    "parallel_only": [_par(2, 2, 16, 16, 6, 2, (8, 100.0), 4.0, 24, 4, 2, 3, mlp=_FF), _par(4, 1, 8, 24, 9, 5, None, 0.0, 16, 7, 3, 2)],
    "one_attention": [_attn(2, 1, 24, 8, 7, 12, 4, mlp=_FF)],
    "one_parallel": [_par(2, 1, 24, 8, 7, 3, (24, 30.0), 3.0, 24, 4, 2, 2)],
    "chain_of_three": [_par(2, 1, 16, 16, 6, 3, (8, 100.0), 0.0, 24, 4, 2, 3), _attn(2, 2, 16, 20, 4, 9, 4), _attn(2, 2, 16, 20, 9, 9, 8, mlp=_FF),
                       _attn(2, 2, 16, 20, 14, 30, 6)],
    "in_turn": [_par(2, 1, 16, 16, 6, 3, (8, 100.0), 6.0, 24, 4, 2, 3, mlp=_FF), _attn(2, 1, 16, 16, 6, 10, 6), _par(2, 1, 16, 16, 6, 3, (8, 100.0), 6.0, 24, 4, 2, 3),
                _attn(2, 1, 16, 16, 6, 10, 6, mlp=_FF)],
}


@pytest.mark.parametrize("order", list(ORDERS))
def test_other_orders_of_layers(tmp_path_factory, order):
    cfg = _config(67, 40, ORDERS[order])
    folder, weights, cfg = _folder(tmp_path_factory, "A", cfg=cfg, seed=3)
    reqs = _requests(cfg["vocab"], [1, 40, 75], seed=1)
    steps = H.cut_mixed(reqs, max_live=3, seed=5, portion_sizes=(2, 3, 5, 8, 17))
    for dtype in ("float32", "bfloat16"):
        _compare(folder, weights, cfg, reqs, steps, dtype, order, slots=3)


def test_residual_stream_after_every_layer(models):
    """The stream after each layer (the model's own trace) against the plain implementation's."""
    from quanta_b200.engine.step import StepEntry
    folder, weights, cfg = models["A"]
    toks = H.random_tokens(29, cfg["vocab"], 3)
    _, layers, _ = P.forward(weights, cfg, toks, return_layers=True)
    eng = _engine(folder, "float32", num_pages=8)
    eng.model.residual_trace = []
    eng.step([StepEntry("a", toks, (0,))], end=["a"])
    assert len(eng.model.residual_trace) == len(cfg["layers"])
    for i, got in enumerate(eng.model.residual_trace):
        assert torch.allclose(got.cpu(), layers[i], atol=2e-4 * float(layers[i].abs().max()), rtol=1e-4), i


def test_token_by_token_equals_whole_prompt(models):
    """Every token alone (the scan's state and the convolution's inputs cross a step at every token, every pooled
    block is closed by a step of one token) against the prompt in one step."""
    for name in ("A", "C"):
        folder, weights, cfg = models[name]
        reqs = _requests(cfg["vocab"], [45], seed=3)
        one = H.cut_tail_decode(reqs, tail=1000)
        whole = H.cut_whole(reqs)
        a = H.replay(_engine(folder, "float32", one, page_size=4), one)
        b = H.replay(_engine(folder, "float32", whole, page_size=4), whole)
        worst, where = _worst(a, b)
        assert worst < 2e-5, (name, worst, where)


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
    side by side: windows pass over decoded tokens, pooled blocks close and come into sight, pages of tokens that
    left every window are given back, all at different steps for the two."""
    folder, weights, cfg = models["E"]
    reqs = _requests(cfg["vocab"], [157, 171], seed=4)
    steps = [{"entries": [{"id": "r0", "tokens": reqs["r0"][:7], "want": [6]}, {"id": "r1", "tokens": reqs["r1"][:21], "want": [20]}],
              "end": []}]
    for i in range(150):
        steps.append({"entries": [{"id": "r0", "tokens": [reqs["r0"][7 + i]], "want": [0]},
                                  {"id": "r1", "tokens": [reqs["r1"][21 + i]], "want": [0]}], "end": []})
    want, _ = _want(weights, cfg, reqs)
    for dtype in ("float32", "bfloat16"):
        # pages for the two requests' full lengths (the pooled rows all stay, and their pages are a share of this
        # count); the token pages are let go as the windows pass and never come near that number
        eng = _engine(folder, dtype, num_pages=44, page_size=8)
        got = H.replay(eng, steps)
        assert eng.stats()["graph_replays"] > 100
        windowed = [g for g in eng.manager.stats()["groups"] if g["window"] is not None]
        assert windowed and all(g["high_water"] <= 12 for g in windowed), windowed
        worst, where = _worst(got, {k: want[k] for k in got})
        assert worst < TOL[dtype], (dtype, worst, where)


def test_slots_and_pages_are_used_again(models):
    """One slot and the pages of one request: five requests one after the other, each starting from a zero state
    and its own pooled blocks although the slot and the pages still hold the last request's numbers."""
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
    plain model with ONE constant or tensor changed (a window one token longer or shorter, a ladder that ends
    elsewhere, no sink, no blending, a block of another size, no cap, unmixed heads, other branch weights, the
    correction left out of the choice, the pass-through experts given weights of zero) is far off: none of them
    is a detail that this test could not see."""
    layers = [_attn(2, 1, 16, 16, 6, 14, 8, scale=0.9, mlp=_moe(3, 2, 2, 16, 8)),
              _par(2, 1, 16, 16, 7, 3, (8, 40.0), 1.5, 24, 4, 2, 3, (0.6, 1.4), scale=1.2, mlp=_moe(3, 2, 2, 16, 8)),
              _attn(2, 1, 16, 16, 9, 20, 6, scale=0.9)]
    folder, weights, cfg = _folder(tmp_path_factory, "A", cfg=_config(50, 48, layers), seed=77)
    weights = dict(weights)
    for i in (0, 1):
        weights[f"l{i}.mlp.correction"] = (weights[f"l{i}.mlp.correction"].float() * 8).to(torch.bfloat16)
    from quanta_b200.weights.safetensors_io import write_safetensors
    write_safetensors(folder / "model.safetensors", weights)
    reqs = _requests(cfg["vocab"], [41], seed=2)
    steps = H.cut_portions(reqs, sizes=(2, 3, 1, 2, 4, 6, 1, 1, 1, 5, 3, 12))
    got = H.replay(_engine(folder, "float32", steps, page_size=4), steps)
    want, margins = _want(weights, cfg, reqs)
    worst, where = _worst(got, want, margins, NEAR_TIE["float32"])
    assert worst < TOL["float32"], (worst, where)

    def other(edit, w=None):
        c = json.loads(json.dumps(cfg))
        if edit is not None:
            edit(c["layers"])
        far, _ = _worst(got, _want(w or weights, c, reqs)[0])
        return far

    def setter(layer, path, value):
        def edit(layers):
            m = layers[layer]["mixer"]
            for key in path[:-1]:
                m = m[key]
            m[path[-1]] = value
        return edit

    changed = {
        "window + 1": other(setter(0, ("mask", "size"), 7)), "window - 1": other(setter(2, ("mask", "size"), 8)),
        "ladder": other(setter(0, ("bias_max",), 6)), "scale": other(setter(0, ("scale",), 0.5)),
        "no blending": other(setter(2, ("v_mix",), False)),
        "left window + 1": other(setter(1, ("left", "mask", "size"), 8)), "block": other(setter(1, ("left", "mask", "pool"), 4)),
        "cap": other(setter(1, ("left", "softcap"), 0.0)), "rotation": other(setter(1, ("left", "rot", "base"), 4.0)),
        "rotated part": other(setter(1, ("left", "rot", "dims"), 4)),
        "branch weights": other(setter(1, ("left_scale",), 1.4)),
        "no sink": other(None, dict(weights, **{"l0.mix.sink": torch.full_like(weights["l0.mix.sink"], -30.0)})),
        "unmixed heads": other(None, dict(weights, **{"l1.mix.left.talk": torch.eye(2).to(torch.bfloat16)})),
        "no correction": other(None, dict(weights, **{"l0.mlp.correction": torch.zeros_like(weights["l0.mlp.correction"])})),
        "one gain": other(None, dict(weights, **{"l1.norm2": weights["l1.norm2"] * 1.5})),
        "conv bias": other(None, dict(weights, **{"l1.mix.right.conv.b": weights["l1.mix.right.conv.b"] * 0})),
    }
    for what, far in changed.items():
        assert far > 30 * TOL["float32"], (what, far)


def test_greedy_generation_through_the_scheduler(models):
    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    folder, weights, cfg = models["A"]
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
