"""Gate: the Puvolix decoder through the entry point gives the plain implementation's tokens and logits.

A small model (norms in three groups; in every layer a softmax attention with convolved q, k, v, rescaled rotation and
head temperatures beside a gated delta rule; a dense feed-forward with biases, input-weighted clamped experts with a
shared expert, and a layer without a feed-forward; a depth-weighted stream; capped logits): greedy tokens of three
prompts fed in portions of 6 beside decoded tokens, pages of 4, two state slots that are used again; then the logits
of one prompt through the step function, whole and token by token."""
# parity-gate: gpu

from __future__ import annotations

import json
import tempfile
from pathlib import Path

from parity._gates import Checks


def _layer(mlp):
    return {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 20, "conv": 2, "scale": 0.3,
                 "rot": {"dims": 8, "base": 100.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 40}}},
        "right": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 12, "conv": 4}}}


CONFIG = {"architecture": "Puvolix", "vocab": 90, "width": 48, "norm": {"eps": 1e-5, "groups": 3}, "logit_softcap": 10.0,
          "layers": [_layer({"kind": "dense", "ff": 40}),
                     _layer({"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 24, "limit": 1.2},
                             "shared": {"ff": 16, "limit": 0.8}}),
                     _layer(None)]}


def run() -> int:
    import torch

    from quanta_b200 import generate
    from quanta_b200.engine.generate import LLM
    from quanta_b200.weights.safetensors_io import write_safetensors
    from tests import helpers as H
    from tests.plain import puvolix_plain as P

    c = Checks("puvolix_generate_test")
    with tempfile.TemporaryDirectory() as d:
        weights = P.draw_weights(CONFIG, seed=5)
        write_safetensors(Path(d) / "model.safetensors", weights)
        (Path(d) / "config.json").write_text(json.dumps(CONFIG))
        llm = LLM(d, dtype="float32", page_size=4, num_pages=40, max_requests=2, max_step_tokens=12, prefill_chunk=6)
        prompts = [H.random_tokens(n, CONFIG["vocab"], 40 + i) for i, n in enumerate((5, 11, 16))]
        got = generate(llm, prompts, max_new_tokens=8, eos_id=[])
        for p, g in zip(prompts, got):
            c.ok(g == P.generate(weights, CONFIG, p, 8), f"greedy tokens of a prompt of {len(p)}")
        c.ok(llm.engine.manager.stats()["live_requests"] == 0, "all slots released")
        reqs = {"a": H.random_tokens(33, CONFIG["vocab"], 7)}
        want = P.forward(weights, CONFIG, reqs["a"])
        for name, steps in (("whole", H.cut_whole(reqs)), ("token by token", H.cut_tail_decode(reqs, tail=1000))):
            rows = H.replay(llm.engine, steps)
            worst = max(float((rows[("a", i)] - want[i]).abs().max()) for i in range(33))
            c.ok(worst < 2e-4 * float(want.abs().max()), f"logits, {name}: {worst}")
        c.ok(torch.isfinite(want).all().item(), "finite logits")
    c.done()
    return 0


if __name__ == "__main__":
    raise SystemExit(run())
