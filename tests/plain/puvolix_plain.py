"""Plain, slow implementation of the Puvolix decoder, one function per mechanism, whole sequences only.

It shares no code with the engine: float torch (float32, or float64 on request) on whatever device the weights
are on, token by token where the design is a recurrence.  ``forward(weights, config, tokens)`` returns the logits
at every position and, on request, the residual stream after every layer.

The design: a token table; layers ``x += n1(mixer(x))`` then ``x += n2(ff(x))`` whose sublayers read the stream
itself and whose norms divide each of ``groups`` equal parts of the vector by that part's own root mean square;
after layer i the stream becomes a learned weighted sum of the embedding output and the results of layers 0..i.
The one mixer, ``parallel``, is half the sum of two RMS-normed branches: grouped-query softmax attention whose
projected q, k, v pass a short causal convolution, with a per-head norm of q and k, a partial rotation whose
frequencies are rescaled by wavelength, and a learned number per head on the scores; and a gated delta rule
(short convolutions with silu, unit queries and keys, a write strength and a decay per head, a per-head output
norm with a silu gate).  Feed-forwards are a gated dense layer with biases, or sigmoid-routed experts whose
routing weight multiplies the expert's input, with clamped gate and up branches, beside a shared expert.  The
head is the grouped norm, an output matrix and a tanh cap on the logits.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
import torch.nn.functional as F


def read_config(model_dir) -> dict:
    return json.loads((Path(model_dir) / "config.json").read_text())


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_norm(x, w, groups: int, eps: float):
    """The vector in ``groups`` equal consecutive parts, each divided by its own root mean square; times ``w``."""
    T, W = x.shape
    return rms(x.view(T, groups, W // groups), eps).reshape(T, W) * w


def causal_conv(u, w):
    """``u`` [T, C], ``w`` [C, taps]: ``y_t = sum_j w[:, j] u_(t - taps + 1 + j)``, zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([u.new_zeros(taps - 1, C), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j] * padded[j: j + T]
    return y


def scaled_frequencies(dims: int, base: float, scaling: dict | None, dtype):
    """``f_i = base^(-2i/dims)``; with ``scaling`` the long wavelengths are slowed down by ``factor``, the short
    ones kept, and those between blended linearly in ``original / wavelength``."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        lam = 2.0 * math.pi / fi
        if lam < orig / high:
            out.append(fi)
        elif lam > orig / low:
            out.append(fi / factor)
        else:
            s = (orig / lam - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=dtype)


def rotate(x, positions, dims: int, freqs):
    """``x`` [T, heads, d]: coordinate i of the first ``dims`` is paired with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    ang = positions.to(x.dtype)[:, None] * freqs.to(x.device, x.dtype)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], -1)


def softmax_attention(w, p: str, h, m: dict, eps: float):
    """The left branch.  ``h`` [T, width]."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if int(m.get("conv") or 0) > 0:
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q = rms(q.view(T, H, D), eps) * w[p + "q.norm"]
    k = rms(k.view(T, G, D), eps) * w[p + "k.norm"]
    v = v.view(T, G, V)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    pos = torch.arange(T, device=h.device)
    if dims:
        f = scaled_frequencies(dims, float(rot["base"]), rot.get("scaling"), h.dtype)
        q, k = rotate(q, pos, dims, f), rotate(k, pos, dims, f)
    out = attend(q, k, v, float(m["scale"]), w[p + "temp"])
    return out.reshape(T, H * V) @ w[p + "o"].T


def attend(q, k, v, scale: float, temp):
    """Causal softmax attention of one sequence: ``q`` [T, H, D], ``k`` [T, G, D], ``v`` [T, G, V], a number per head
    (``temp`` [H]) on the scaled scores -> [T, H, V]."""
    T, H, _ = q.shape
    G = k.shape[1]
    pos = torch.arange(T, device=q.device)
    mask = pos[None, :] <= pos[:, None]
    out = q.new_zeros(T, H, v.shape[2])
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * scale * temp[head]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(s, -1) @ v[:, g]
    return out


def gated_delta_rule(w, p: str, h, m: dict, eps: float):
    """The right branch, token by token.  State ``S`` [dim, vdim] per head."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if int(m.get("conv") or 0) > 0:
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q, k, v = F.silu(q).view(T, G, D), F.silu(k).view(T, G, D), F.silu(v).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                                   # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o, _ = delta_recurrence(q, k, v, decay, beta)
    o = rms(o, eps) * w[p + "norm"]
    o = o * F.silu(h @ w[p + "g"].T).view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].T


def delta_recurrence(q, k, v, decay, beta, S=None):
    """``q``, ``k`` [T, G, D]; ``v`` [T, H, V]; ``decay``, ``beta`` [T, H].  Per head, in this order:
    ``S <- decay S``; ``u = beta (v - S^T k)``; ``S <- S + k u^T``; ``o = S^T q``.  Returns (o [T, H, V], S)."""
    T, H, V = v.shape
    G, D = k.shape[1], k.shape[2]
    S = v.new_zeros(H, D, V) if S is None else S.clone()
    o = v.new_zeros(T, H, V)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            o[t, head] = S[head].T @ q[t, g]
    return o, S


def parallel_mixer(w, p: str, h, m: dict, eps: float):
    left = softmax_attention(w, p + "left.", h, m["left"], eps)
    right = gated_delta_rule(w, p + "right.", h, m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


def dense_ff(w, p: str, h):
    g = h @ w[p + "gate"].T + w[p + "gate.b"]
    u = h @ w[p + "up"].T + w[p + "up.b"]
    return (F.silu(g) * u) @ w[p + "down"].T + w[p + "down.b"]


def clamped_expert(w, p: str, h, limit: float):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def router_choice(w, p: str, h, top: int):
    """(experts [T, top], their sigmoid scores [T, top], margin [T]); equal scores go to the lower index.  The
    margin is the gap between the last chosen score and the best one left out (a choice rounding could turn)."""
    s = torch.sigmoid(h.float() @ w[p + "router"].float().T)
    ranked = torch.sort(s, dim=-1, descending=True, stable=True)
    order = ranked.indices[:, :top]
    margin = ranked.values[:, top - 1] - ranked.values[:, top] if s.shape[1] > top else torch.full((h.shape[0],), 1e9)
    return order, torch.gather(s, 1, order), margin


def routed_ff(w, p: str, h, mlp: dict, chosen=None):
    """``chosen`` [T, top]: take these experts (with their own scores) instead of the router's choice."""
    top, limit = int(mlp["router"]["top"]), float(mlp["expert"]["limit"])
    idx, score, margin = router_choice(w, p, h, top)
    if chosen is not None:
        idx = chosen.to(idx.device).long()
        score = torch.gather(torch.sigmoid(h.float() @ w[p + "router"].float().T), 1, idx)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            y[t] = y[t] + clamped_expert(w, f"{p}e{e}.", (score[t, c].to(h.dtype) * h[t])[None], limit)[0]
    shared = mlp.get("shared")
    if shared is not None:
        y = y + clamped_expert(w, p + "shared.", h, float(shared["limit"]))
    return y, idx, margin


def forward(weights: dict, config: dict, tokens, dtype=torch.float32, chosen=None, details: bool = False):
    """Logits ``[T, vocab]`` of one whole sequence.  ``chosen``: one ``[T, top]`` tensor per routed layer, in layer
    order, that replaces the router's choice.  ``details``: also a dictionary with ``layers`` (the stream that goes
    on after every layer), ``results`` (every layer's own result, before the weighted sum) and ``routing`` (per
    routed layer the chosen experts and the margin of the choice)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"].get("groups") or 1)
    ids = torch.as_tensor(tokens, dtype=torch.long, device=w["embed"].device)
    x = w["embed"][ids]
    results, after, routing = [x], [], []
    chosen = list(chosen) if chosen is not None else None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + grouped_norm(parallel_mixer(w, p + "mix.", x, layer["mixer"], eps), w[p + "norm1"], groups, eps)
        mlp = layer.get("mlp")
        if mlp is not None and mlp.get("kind") == "dense":
            x = x + grouped_norm(dense_ff(w, p + "mlp.", x), w[p + "norm2"], groups, eps)
        elif mlp is not None:
            y, idx, margin = routed_ff(w, p + "mlp.", x, mlp, chosen.pop(0) if chosen is not None else None)
            routing.append((idx, margin))
            x = x + grouped_norm(y, w[p + "norm2"], groups, eps)
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        after.append(x)
    x = grouped_norm(x, w["final.norm"], groups, eps)
    logits = x @ w["head"].T
    cap = float(config.get("logit_softcap") or 0.0)
    if cap:
        logits = cap * torch.tanh(logits / cap)
    if details:
        return logits, {"layers": torch.stack(after), "results": torch.stack(results[1:]), "routing": routing}
    return logits


def generate(weights: dict, config: dict, prompt, n_new: int) -> list[int]:
    """Greedy continuation, the whole sequence run again for every token."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(weights, config, toks)[-1].argmax()))
    return toks[len(prompt):]


# ---- random weights of a configuration ----------------------------------------------------------------------
def tensor_shapes(config: dict) -> dict:
    W, V = int(config["width"]), int(config["vocab"])
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        shapes[p + "norm1"] = (W,)
        shapes[p + "dwa"] = (i + 2,)
        l, r = layer["mixer"]["left"], layer["mixer"]["right"]
        H, G, D, Vd = int(l["heads"]), int(l["kv_heads"]), int(l["dim"]), int(l["vdim"])
        q = p + "mix.left."
        shapes.update({q + "q": (H * D, W), q + "k": (G * D, W), q + "v": (G * Vd, W), q + "o": (W, H * Vd),
                       q + "q.norm": (D,), q + "k.norm": (D,), q + "temp": (H,), q + "out": (W,)})
        taps = int(l.get("conv") or 0)
        if taps:
            shapes.update({q + "q.conv": (H * D, taps), q + "k.conv": (G * D, taps), q + "v.conv": (G * Vd, taps)})
        H, G, D, Vd = int(r["heads"]), int(r["kv_heads"]), int(r["dim"]), int(r["vdim"])
        q = p + "mix.right."
        shapes.update({q + "q": (G * D, W), q + "k": (G * D, W), q + "v": (H * Vd, W), q + "g": (H * Vd, W),
                       q + "b": (H, W), q + "a": (H, W), q + "A_log": (H,), q + "dt_bias": (H,), q + "norm": (Vd,),
                       q + "o": (W, H * Vd), q + "out": (W,)})
        taps = int(r.get("conv") or 0)
        if taps:
            shapes.update({q + "q.conv": (G * D, taps), q + "k.conv": (G * D, taps), q + "v.conv": (H * Vd, taps)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (W,)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            F_ = int(mlp["ff"])
            shapes.update({q + "gate": (F_, W), q + "gate.b": (F_,), q + "up": (F_, W), q + "up.b": (F_,),
                           q + "down": (W, F_), q + "down.b": (W,)})
        else:
            F_ = int(mlp["expert"]["ff"])
            shapes[q + "router"] = (int(mlp["router"]["experts"]), W)
            for e in range(int(mlp["router"]["experts"])):
                shapes.update({f"{q}e{e}.gate": (F_, W), f"{q}e{e}.up": (F_, W), f"{q}e{e}.down": (W, F_)})
            if mlp.get("shared") is not None:
                S = int(mlp["shared"]["ff"])
                shapes.update({q + "shared.gate": (S, W), q + "shared.up": (S, W), q + "shared.down": (W, S)})
    return shapes


def draw_weights(config: dict, seed: int) -> dict:
    """bfloat16 tensors by name, drawn so that no constant of the design is near neutral: gains away from one,
    taps of every age, weights of the depth sum of both signs, decays between slow and fast."""
    g = torch.Generator().manual_seed(seed)
    uni = lambda shape, lo, hi: torch.empty(shape).uniform_(lo, hi, generator=g)  # noqa: E731
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith(".conv"):
            t = uni(shape, -0.5, 0.5)
            t[:, -1] += 1.0
        elif leaf in ("norm1", "norm2", "norm", "out") or name == "final.norm":
            t = uni(shape, 0.6, 1.4)
        elif leaf == "temp":
            t = uni(shape, 0.5, 2.0)
        elif leaf == "dwa":
            t = uni(shape, -0.4, 0.4)
            t[-1] += 1.0
        elif leaf == "A_log":
            t = uni(shape, -2.0, 1.0)
        elif leaf == "dt_bias":
            t = uni(shape, -1.0, 1.0)
        elif leaf == "b" and len(shape) == 1:
            t = uni(shape, -0.3, 0.3)
        elif leaf == "router":
            t = torch.randn(shape, generator=g) * 2.0 / math.sqrt(shape[1])
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * 1.5 / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out
