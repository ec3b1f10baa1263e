"""Tarulix decoder: from its configuration to a model specification.

A token table; layers ``l<i>.`` whose sublayers read the residual stream itself and whose OUTPUT is normed before
it joins the stream, ``x += g1 * rms(mixer(x))`` and, where the layer has a feed-forward, ``x += g2 * rms(ff(x))``
(each norm has one number as its gain).  Two kinds of mixer: ``attention`` (sliding-window grouped-query attention
with projection biases, unit-RMS queries and keys, a learned bias by bucketed distance, a sink in the softmax
denominator, values blended with those of the first such layer, no rotation) and ``parallel`` (the weighted sum of
a rotary sliding-window attention that also reads the means of blocks of older tokens, caps its scores with a
tanh and mixes the heads' softmax weights, and a selective state-space scan).  Feed-forwards are routed gated
experts with a softmax router, experts that hand their input through, and a shared expert.  The head is the
model's norm and an output matrix of its own.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tarulix import DEFAULT_BIAS_ROWS, TarulixConfig
from ..parts.spec import ModelSpec

BLEND_KEY = "tarulix_first_values"


def _attention_names(mix: str) -> dict:
    return {"q": mix + "q", "k": mix + "k", "v": mix + "v", "o": mix + "o", "q_b": mix + "q.b", "k_b": mix + "k.b",
            "v_b": mix + "v.b", "o_b": mix + "o.b", "rel": mix + "rel", "sink": mix + "sink", "talk": mix + "talk",
            "vmix": mix + "vmix"}


def biased_attention(cfg: TarulixConfig, i: int, m: dict, first_blend: int | None) -> tuple[str, dict]:
    blend = None
    if m.get("v_mix"):
        blend = "source" if first_blend == i else "blend"
    rows = m.get("bias_rows")
    if rows is None:                       # no checkpoint: as many rows as the ladder's end allows
        rows = DEFAULT_BIAS_ROWS
        while rows > 2 and float(m["bias_max"]) <= rows // 2:
            rows //= 2
    return ("window_attention", dict(
        hidden_size=cfg.width, n_q_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
        value_dim=int(m["vdim"]), scale=float(m["scale"]), window=int(m["mask"]["size"]), norm_eps=cfg.norm_eps,
        names=_attention_names(f"l{i}.mix."), position=("none", {}), unit_qk=True, biases=True,
        distance_bias=(int(rows), float(m["bias_max"])), sink=True,
        value_blend=blend, blend_key=BLEND_KEY))


def pooled_attention(cfg: TarulixConfig, i: int, m: dict) -> tuple[str, dict]:
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    position = ("partial_rotary", dict(head_dim=int(m["dim"]), rotary_dim=dims, theta=float(rot["base"]))) if dims \
        else ("none", {})
    return ("window_attention", dict(
        hidden_size=cfg.width, n_q_heads=int(m["heads"]), n_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
        value_dim=int(m["vdim"]), scale=float(m["scale"]), window=int(m["mask"]["size"]), norm_eps=cfg.norm_eps,
        names=_attention_names(f"l{i}.mix.left."), position=position, unit_qk=True, biases=True,
        softcap=float(m.get("softcap") or 0.0), pool=int(m["mask"].get("pool") or 0), talk=True))


def scan(cfg: TarulixConfig, i: int, m: dict) -> tuple[str, dict]:
    p = f"l{i}.mix.right."
    return ("selective_scan", dict(
        hidden_size=cfg.width, inner=int(m["inner"]), n_state=int(m["state"]), dt_rank=int(m["dt_rank"]),
        conv_taps=int(m["conv"]),
        names={"in": p + "in", "conv": p + "conv", "conv_b": p + "conv.b", "x": p + "x", "dt": p + "dt",
               "dt_b": p + "dt.b", "A_log": p + "A_log", "D": p + "D", "o": p + "o"}))


def routed_experts(cfg: TarulixConfig, i: int, mlp: dict) -> tuple[str, dict]:
    p = f"l{i}.mlp."
    router, shared = mlp["router"], mlp.get("shared")
    return ("softmax_shared_experts", dict(
        hidden_size=cfg.width, expert_size=int((mlp.get("expert") or {}).get("ff", 0)),
        n_experts=int(router["experts"]), n_identity=int(router.get("identity") or 0), top_k=int(router["top"]),
        shared_size=0 if shared is None else int(shared["ff"]), use_bias=True,
        names={"gate": p + "router", "bias": p + "correction", "w1": p + "e{e}.gate", "w3": p + "e{e}.up",
               "w2": p + "e{e}.down", "shared_gate": p + "shared.gate", "shared_up": p + "shared.up",
               "shared_down": p + "shared.down"}))


def layer_choice(cfg: TarulixConfig, i: int, first_blend: int | None) -> tuple[str, dict]:
    layer = cfg.layers[i]
    m = layer.mixer
    gain = lambda n: ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=f"l{i}.{n}", scalar_gain=True))  # noqa: E731
    if layer.type == "attention":
        mixer = biased_attention(cfg, i, m, first_blend)
    else:
        mixer = ("parallel_mixers", dict(left=pooled_attention(cfg, i, m["left"]), right=scan(cfg, i, m["right"]),
                                         left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"])))
    params = dict(hidden_size=cfg.width, mixer=mixer, mixer_norm=("none", dict(width=cfg.width)),
                  mixer_post_norm=gain("norm1"))
    if layer.mlp is not None:
        params.update(feed_forward=routed_experts(cfg, i, layer.mlp),
                      feed_forward_norm=("none", dict(width=cfg.width)), feed_forward_post_norm=gain("norm2"))
    return ("sandwich_norm", params)


def build_spec(cfg: TarulixConfig) -> ModelSpec:
    blending = [i for i, l in enumerate(cfg.layers) if l.type == "attention" and l.mixer.get("v_mix")]
    first_blend = blending[0] if blending else None
    final_norm = ("rms_norm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name="final.norm", scalar_gain=True))
    # a checkpoint may hold a blending fraction for attention layers that blend nothing (the first of the chain and
    # layers outside it)
    unused = tuple(f"l{i}.mix.vmix" for i, l in enumerate(cfg.layers)
                   if l.type == "attention" and (i == first_blend or not l.mixer.get("v_mix")))
    return ModelSpec(
        name="Tarulix", vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
        layers=[layer_choice(cfg, i, first_blend) for i in range(len(cfg.layers))],
        final_norm=final_norm, head_name="head", tied_head=False, ignorable_names=unused)


ARCHITECTURE = register_architecture(["Tarulix", "tarulix"], TarulixConfig, build_spec)
