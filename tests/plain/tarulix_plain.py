"""Plain, slow implementation of the Tarulix decoder, one function per mechanism, whole sequences only.

It shares no code with the engine: float torch (float32, or float64 on request) on whatever device the weights
are on, token by token where the design is a recurrence.  ``forward(weights, config, tokens)`` returns the logits
at every position and, on request, the residual stream after every layer.

The design: a token table; layers ``x += g1 * rms(mixer(x))`` then ``x += g2 * rms(ff(x))`` (sublayers read the
stream itself; the norm has one number as its gain); two mixers, ``attention`` (grouped-query softmax attention
with projection biases, unit-RMS queries and keys, a learned bias by bucketed distance, a sliding window, a sink
in the softmax denominator and values blended with those of the first such layer) and ``parallel`` (the weighted
sum of a rotary sliding-window attention that also sees the means of blocks of older tokens, caps its scores by
a tanh and mixes the heads' softmax weights, and a selective state-space scan); routed experts with a softmax
router, experts that hand their input through, and a shared expert; a final norm and an output matrix.
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


def scalar_norm(x, g, eps):
    """``g * x / sqrt(mean(x^2) + eps)`` with one number ``g`` for all coordinates."""
    return rms(x, eps) * g


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Bucket of the distance ``n >= 0`` in a table of ``rows`` rows: the first half of the rows are the
    distances themselves, the second half is a logarithmic ladder that reaches the last row at ``far``."""
    half = rows // 2
    if n < half:
        return n
    step = math.log(n / half) / math.log(far / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(step)))


def unit_heads(x, heads: int, eps: float):
    """``x`` [T, heads * d] -> [T, heads, d], every head divided by its root mean square."""
    T = x.shape[0]
    return rms(x.view(T, heads, -1), eps)


def rotate_half(x, positions, dims: int, base: float):
    """``x`` [T, heads, d]: the first ``dims`` coordinates of every head are rotated in pairs ``(i, i + dims/2)``
    by the angle ``position * base^(-2i/dims)``; the rest passes."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype, device=x.device)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]                   # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def biased_sink_attention(x, w, m: dict, eps: float, v_first=None):
    """The ``attention`` mixer on a whole sequence.  ``w``: tensors by short name (q, q.b, k, k.b, v, v.b, rel,
    vmix, sink, o, o.b).  ``v_first``: the values [T, G, vd] of the first layer of the blending chain, or None
    when this layer is that first one (or blends nothing).  Returns (output [T, width], this layer's values)."""
    T = x.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window, scale = int(m["mask"]["size"]), float(m["scale"])
    q = unit_heads(x @ w["q"].T + w["q.b"], H, eps)
    k = unit_heads(x @ w["k"].T + w["k.b"], G, eps)
    v = (x @ w["v"].T + w["v.b"]).view(T, G, vd)
    if v_first is not None:
        lam = w["vmix"]
        v = (1 - lam) * v + lam * v_first
    rel = w["rel"]
    rows, far = rel.shape[0], float(m["bias_max"])
    out = torch.zeros((T, H, vd), dtype=x.dtype, device=x.device)
    for i in range(T):
        lo = max(0, i - window + 1)
        js = list(range(lo, i + 1))
        buckets = torch.tensor([distance_bucket(i - j, rows, far) for j in js], device=x.device)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale + rel[buckets, h]
            top = torch.maximum(s.max(), w["sink"][h])
            e = torch.exp(s - top)
            p = e / (e.sum() + torch.exp(w["sink"][h] - top))
            out[i, h] = p @ v[lo:i + 1, g]
    return out.reshape(T, H * vd) @ w["o"].T + w["o.b"], v


def pooled_window_attention(x, w, m: dict, eps: float):
    """The attention half of the ``parallel`` mixer on a whole sequence.  ``w``: q, q.b, k, k.b, v, v.b, talk, o,
    o.b.  Position i reads the last ``size`` tokens and, for every block of ``pool`` tokens that ended at or
    before ``i - size``, the mean key and mean value of the block."""
    T = x.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, P = int(m["mask"]["size"]), int(m["mask"]["pool"])
    scale, cap = float(m["scale"]), float(m["softcap"])
    pos = torch.arange(T, device=x.device)
    q = (x @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (x @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (x @ w["v"].T + w["v.b"]).view(T, G, vd)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rms(rotate_half(q, pos, int(rot["dims"]), float(rot["base"])), eps)
    k = rms(rotate_half(k, pos, int(rot["dims"]), float(rot["base"])), eps)
    n_blocks = T // P
    if n_blocks:
        kp = k[: n_blocks * P].view(n_blocks, P, G, d).mean(1)
        vp = v[: n_blocks * P].view(n_blocks, P, G, vd).mean(1)
    out = torch.zeros((T, H, vd), dtype=x.dtype, device=x.device)
    for i in range(T):
        lo = max(0, i - size + 1)
        seen = max(0, (i - size + 1) // P)              # blocks b with b * P + P - 1 <= i - size
        weights, values = [], []
        for g in range(G):
            keys = k[lo:i + 1, g] if not seen else torch.cat([kp[:seen, g], k[lo:i + 1, g]])
            values.append(v[lo:i + 1, g] if not seen else torch.cat([vp[:seen, g], v[lo:i + 1, g]]))
            for h in range(g * (H // G), (g + 1) * (H // G)):
                s = (keys @ q[i, h]) * scale
                s = cap * torch.tanh(s / cap)
                weights.append(torch.softmax(s, -1))
        mixed = w["talk"] @ torch.stack(weights)        # [H, keys]: head h takes sum_g talk[h, g] weights_g
        for h in range(H):
            out[i, h] = mixed[h] @ values[h // (H // G)]
    return out.reshape(T, H * vd) @ w["o"].T + w["o.b"]


def causal_conv(x, taps_w, bias):
    """``x`` [T, C]; ``taps_w`` [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, C), dtype=x.dtype, device=x.device), x])
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + padded[j: j + T] * taps_w[:, j]
    return y + bias


def selective_scan(x, w, m: dict):
    """The state-space half of the ``parallel`` mixer on a whole sequence, token by token.  ``w``: in, conv,
    conv.b, x, dt, dt.b, A_log, D, o."""
    T = x.shape[0]
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = x @ w["in"].T
    u, z = xz[:, :inner], xz[:, inner:]
    u = F.silu(causal_conv(u, w["conv"], w["conv.b"]))
    proj = u @ w["x"].T
    dt, B, C = proj[:, :R], proj[:, R: R + N], proj[:, R + N: R + 2 * N]
    dt = F.softplus(dt @ w["dt"].T + w["dt.b"])                              # [T, inner]
    A = -torch.exp(w["A_log"])                                               # [inner, N]
    S = torch.zeros((inner, N), dtype=x.dtype, device=x.device)
    y = torch.zeros((T, inner), dtype=x.dtype, device=x.device)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w["D"] * u[t]
    return (y * F.silu(z)) @ w["o"].T


def gated_expert(h, gate, up, down):
    return (F.silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_ff(h, w, m: dict, chosen=None):
    """Softmax over all router outputs; the ``top`` largest of ``score + correction`` are chosen (lower index
    on a tie); the weights are the chosen scores as they are.  The last ``identity`` router outputs stand for
    experts that return their input.  A shared expert is added.  Returns (output, chosen [T, top], margin [T])."""
    E, I, top = int(m["router"]["experts"]), int(m["router"].get("identity", 0)), int(m["router"]["top"])
    s = torch.softmax(h @ w["router"].T, -1)
    choice = s + w["correction"]
    order = torch.sort(choice, dim=-1, descending=True, stable=True)
    idx = order.indices[:, :top]
    margin = (order.values[:, top - 1] - order.values[:, top]) if E + I > top else torch.full_like(s[:, 0], 1e9)
    if chosen is not None:
        idx = torch.as_tensor(chosen, dtype=torch.long, device=h.device)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            y = h[t] if e >= E else gated_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
            out[t] += s[t, e] * y
    if m.get("shared") is not None:
        out = out + gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out, idx, margin


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(weights: dict, cfg: dict, tokens, return_layers: bool = False, chosen=None):
    """Logits [T, vocab] of one whole sequence; with ``return_layers`` also the stream after every layer and the
    experts every routed layer chose.  ``chosen``: per routed layer, experts to take instead of choosing."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long, device=weights["embed"].device)
    x = weights["embed"][ids]
    v_first, layers, picks, routed = None, [], [], 0
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            blend = bool(m.get("v_mix"))
            y, v = biased_sink_attention(x, sub(weights, p + "mix."), m, eps, v_first if blend else None)
            if blend and v_first is None:
                v_first = v
        elif layer["type"] == "parallel":
            left = pooled_window_attention(x, sub(weights, p + "mix.left."), m["left"], eps)
            right = selective_scan(x, sub(weights, p + "mix.right."), m["right"])
            y = float(m["left_scale"]) * left + float(m["right_scale"]) * right
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + scalar_norm(y, weights[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y, idx, _ = routed_ff(x, sub(weights, p + "mlp."), layer["mlp"], None if chosen is None else chosen[routed])
            routed += 1
            picks.append(idx)
            x = x + scalar_norm(y, weights[p + "norm2"], eps)
        layers.append(x.clone())
    logits = scalar_norm(x, weights["final.norm"], eps) @ weights["head"].T
    return (logits, layers, picks) if return_layers else logits
