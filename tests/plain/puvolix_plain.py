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
    out = h.new_zeros(T, H, V)
    mask = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"]) * w[p + "temp"][head]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


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
    S = h.new_zeros(H, D, V)
    o = h.new_zeros(T, H, V)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, g])
            S[head] = S[head] + torch.outer(k[t, g], u)
            o[t, head] = S[head].T @ q[t, g]
    o = rms(o, eps) * w[p + "norm"]
    o = o * F.silu(h @ w[p + "g"].T).view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].T


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
    """(experts [T, top], their sigmoid scores [T, top]); equal scores go to the lower index."""
    s = torch.sigmoid(h.float() @ w[p + "router"].float().T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def routed_ff(w, p: str, h, mlp: dict):
    top, limit = int(mlp["router"]["top"]), float(mlp["expert"]["limit"])
    idx, score = router_choice(w, p, h, top)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            y[t] = y[t] + clamped_expert(w, f"{p}e{e}.", (score[t, c].to(h.dtype) * h[t])[None], limit)[0]
    shared = mlp.get("shared")
    if shared is not None:
        y = y + clamped_expert(w, p + "shared.", h, float(shared["limit"]))
    return y


def feed_forward(w, p: str, h, mlp: dict):
    return dense_ff(w, p, h) if mlp.get("kind") == "dense" else routed_ff(w, p, h, mlp)


def forward(weights: dict, config: dict, tokens, dtype=torch.float32, with_layers: bool = False,
            before_average: bool = False):
    """Logits ``[T, vocab]`` of one whole sequence; with ``with_layers`` also the stream after every layer
    (``before_average``: each layer's own result instead of what goes on to the next)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"].get("groups", 1))
    ids = torch.as_tensor(tokens, dtype=torch.long, device=w["embed"].device)
    x = w["embed"][ids]
    results = [x]
    trace = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + grouped_norm(parallel_mixer(w, p + "mix.", x, layer["mixer"], eps), w[p + "norm1"], groups, eps)
        if layer.get("mlp") is not None:
            x = x + grouped_norm(feed_forward(w, p + "mlp.", x, layer["mlp"]), w[p + "norm2"], groups, eps)
        results.append(x)
        if before_average:
            trace.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        if not before_average:
            trace.append(x)
    x = grouped_norm(x, w["final.norm"], groups, eps)
    logits = x @ w["head"].T
    cap = float(config.get("logit_softcap") or 0.0)
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(trace)) if with_layers else logits
