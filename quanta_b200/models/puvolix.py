"""Puvolix decoder: from its configuration to a model specification.

A token table; layers ``l<i>.`` whose sublayers read the residual stream itself and whose OUTPUT is normed in groups
before it joins the stream, ``x += n1(mixer(x))`` and, where the layer has a feed-forward, ``x += n2(ff(x))``; after
layer i the stream becomes ``sum_j dwa_i[j] X_j`` over the embedding output ``X_0`` and the results ``X_1 .. X_(i+1)``
of the layers so far.  The mixer, ``parallel``, is half the sum of two branches that are each RMS-normed over the
width first: grouped-query softmax attention (a short convolution on the projected q, k, v; a per-head norm of q
and k; a partial rotation with frequencies rescaled by wavelength; a learned number per head on the scores) and a
gated delta rule (short convolutions with silu, unit q and k, a decay and a write strength per head, a per-head
output norm with a silu gate).  Feed-forwards are a gated dense layer with biases, or sigmoid-routed experts whose
routing weight multiplies the expert's input, with clamped branches, beside a shared expert.  The head is the
grouped norm, an output matrix of its own and a tanh cap.
"""

from __future__ import annotations

from ..config.puvolix import PuvolixConfig
from ..config.registry import register_architecture
from ..parts.spec import ModelSpec

# what the design fixes
BRANCH_WEIGHT = 0.5            # the mixer is half the sum of its two normed branches
UNIT_EPS = 1e-6                # under the root that makes the recurrence's q and k unit vectors
EXPERT_ALPHA = 1.702           # the experts' gate branch is g * sigmoid(EXPERT_ALPHA * g)


def softmax_branch(cfg: PuvolixConfig, i: int, m: dict) -> tuple[str, dict]:
    p = f"l{i}.mix.left."
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    position = ("none", {})
    if dims:
        sc = rot.get("scaling")
        scaling = None if sc is None else (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
        position = ("partial_rotary", dict(head_dim=int(m["dim"]), rotary_dim=dims, theta=float(rot["base"]),
                                           wavelength_scaling=scaling))
    taps = int(m.get("conv") or 0)
    names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
             "head_temperature": p + "temp"}
    if taps:
        names.update({"q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv"})
    return ("gqa_attention", dict(
        hidden_size=cfg.width, n_q_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
        value_dim=int(m["vdim"]), scale=float(m["scale"]), position=position, qk_norm="per_head",
        qk_norm_eps=cfg.norm_eps, names=names, float32_output=True, conv_taps=taps, float32_weights=True))


def delta_branch(cfg: PuvolixConfig, i: int, m: dict) -> tuple[str, dict]:
    p = f"l{i}.mix.right."
    taps = int(m.get("conv") or 0)
    names = {k: p + k for k in ("q", "k", "v", "g", "b", "a", "A_log", "dt_bias", "norm", "o")}
    if taps:
        names.update({"q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv"})
    return ("gated_delta_rule", dict(
        hidden_size=cfg.width, n_heads=int(m["heads"]), n_groups=int(m["kv_heads"]), dim=int(m["dim"]),
        value_dim=int(m["vdim"]), conv_taps=taps, q_scale=float(int(m["dim"]) ** -0.5), unit_eps=UNIT_EPS,
        norm_eps=cfg.norm_eps, names=names))


def feed_forward(cfg: PuvolixConfig, i: int, mlp: dict) -> tuple[str, dict]:
    p = f"l{i}.mlp."
    if mlp["kind"] == "dense":
        return ("gated_dense", dict(hidden_size=cfg.width, inner_size=int(mlp["ff"]), biases=True,
                                    names={"gate": p + "gate", "up": p + "up", "down": p + "down", "gate_b": p + "gate.b",
                                           "up_b": p + "up.b", "down_b": p + "down.b"}))
    router, expert, shared = mlp["router"], mlp["expert"], mlp.get("shared")
    return ("input_weighted_experts", dict(
        hidden_size=cfg.width, expert_size=int(expert["ff"]), n_experts=int(router["experts"]), top_k=int(router["top"]),
        limit=float(expert["limit"]), alpha=EXPERT_ALPHA,
        shared_size=0 if shared is None else int(shared["ff"]),
        shared_limit=0.0 if shared is None else float(shared["limit"]),
        names={"gate": p + "router", "w1": p + "e{e}.gate", "w3": p + "e{e}.up", "w2": p + "e{e}.down",
               "shared_gate": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down"}))


def layer_choice(cfg: PuvolixConfig, i: int) -> tuple[str, dict]:
    layer = cfg.layers[i]
    m = layer.mixer
    stream_norm = lambda n: ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=n, groups=cfg.norm_groups))  # noqa: E731
    branch_norm = lambda n: ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=n))  # noqa: E731
    mixer = ("parallel_mixers", dict(left=softmax_branch(cfg, i, m["left"]), right=delta_branch(cfg, i, m["right"]),
                                     left_scale=BRANCH_WEIGHT, right_scale=BRANCH_WEIGHT,
                                     left_norm=branch_norm(f"l{i}.mix.left.out"),
                                     right_norm=branch_norm(f"l{i}.mix.right.out")))
    inner = dict(hidden_size=cfg.width, mixer=mixer, mixer_norm=("none", dict(width=cfg.width)),
                 mixer_post_norm=stream_norm(f"l{i}.norm1"))
    if layer.mlp is not None:
        inner.update(feed_forward=feed_forward(cfg, i, layer.mlp), feed_forward_norm=("none", dict(width=cfg.width)),
                     feed_forward_post_norm=stream_norm(f"l{i}.norm2"))
    return ("depth_weighted", dict(hidden_size=cfg.width, inner=("sandwich_norm", inner), index=i,
                                   depth=len(cfg.layers), weights_name=f"l{i}.dwa"))


def build_spec(cfg: PuvolixConfig) -> ModelSpec:
    final_norm = ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name="final.norm", groups=cfg.norm_groups))
    head = ("linear", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, norm=final_norm, weight_name="head",
                           tied_to=None, softcap=cfg.logit_softcap))
    # a checkpoint may hold the second norm's gain of a layer that has no feed-forward
    unused = tuple(f"l{i}.norm2" for i, l in enumerate(cfg.layers) if l.mlp is None)
    return ModelSpec(
        name="Puvolix", vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
        layers=[layer_choice(cfg, i) for i in range(len(cfg.layers))],
        final_norm=final_norm, head_name="head", tied_head=False, head=head, ignorable_names=unused)


ARCHITECTURE = register_architecture(["Puvolix", "puvolix"], PuvolixConfig, build_spec)
