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


def sink_softmax(s, sink):
    """Softmax weights of the scores ``s`` [keys] when the denominator holds one more term, ``exp(sink)``."""
    top = torch.maximum(s.max(), sink)
    e = torch.exp(s - top)
    return e / (e.sum() + torch.exp(sink - top))


def biased_sink_rows(q, k, v, window: int, scale: float, rel, far: float, sink):
    """``q`` [T, H, d], ``k`` [T, G, d], ``v`` [T, G, vd] of one sequence from its start: position i reads the
    positions ``i - window + 1 .. i``; ``rel`` [rows, H] is added by bucketed distance, ``sink`` [H] joins the
    denominator.  Returns [T, H, vd]."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype, device=q.device)
    for i in range(T):
        lo = max(0, i - window + 1)
        buckets = torch.tensor([distance_bucket(i - j, rel.shape[0], far) for j in range(lo, i + 1)], device=q.device)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale + rel[buckets, h]
            out[i, h] = sink_softmax(s, sink[h]) @ v[lo:i + 1, g]
    return out


def biased_sink_attention(x, w, m: dict, eps: float, v_first=None):
    """The ``attention`` mixer on a whole sequence.  ``w``: tensors by short name (q, q.b, k, k.b, v, v.b, rel,
    vmix, sink, o, o.b).  ``v_first``: the values [T, G, vd] of the first layer of the blending chain, or None
    when this layer is that first one (or blends nothing).  Returns (output [T, width], this layer's values)."""
    T = x.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_heads(x @ w["q"].T + w["q.b"], H, eps)
    k = unit_heads(x @ w["k"].T + w["k.b"], G, eps)
    v = (x @ w["v"].T + w["v.b"]).view(T, G, vd)
    if v_first is not None:
        lam = w["vmix"]
        v = (1 - lam) * v + lam * v_first
    out = biased_sink_rows(q, k, v, int(m["mask"]["size"]), float(m["scale"]), w["rel"], float(m["bias_max"]), w["sink"])
    return out.reshape(T, H * vd) @ w["o"].T + w["o.b"], v


def pooled_rows(q, k, v, size: int, P: int, scale: float, cap: float, talk):
    """``q`` [T, H, d], ``k`` [T, G, d], ``v`` [T, G, vd] of one sequence from its start.  Position i reads the last
    ``size`` tokens and, for every block of ``P`` tokens that ended at or before ``i - size``, the mean key and
    mean value of the block; scores are capped by a tanh (``cap`` 0: not), one softmax over blocks and tokens,
    then head h takes ``sum_g talk[h, g] weights_g`` (``talk`` None: its own) on the values of its kv head."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    n_blocks = T // P if P else 0
    if n_blocks:
        kp = k[: n_blocks * P].view(n_blocks, P, G, -1).mean(1)
        vp = v[: n_blocks * P].view(n_blocks, P, G, -1).mean(1)
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype, device=q.device)
    for i in range(T):
        lo = max(0, i - size + 1)
        seen = max(0, (i - size + 1) // P) if P else 0     # blocks b with b * P + P - 1 <= i - size
        weights, values = [], []
        for g in range(G):
            keys = k[lo:i + 1, g] if not seen else torch.cat([kp[:seen, g], k[lo:i + 1, g]])
            values.append(v[lo:i + 1, g] if not seen else torch.cat([vp[:seen, g], v[lo:i + 1, g]]))
            for h in range(g * (H // G), (g + 1) * (H // G)):
                s = (keys @ q[i, h]) * scale
                if cap:
                    s = cap * torch.tanh(s / cap)
                weights.append(torch.softmax(s, -1))
        mixed = torch.stack(weights)
        if talk is not None:
            mixed = talk @ mixed                        # [H, keys]: head h takes sum_g talk[h, g] weights_g
        for h in range(H):
            out[i, h] = mixed[h] @ values[h // (H // G)]
    return out


def pooled_window_attention(x, w, m: dict, eps: float):
    """The attention half of the ``parallel`` mixer on a whole sequence.  ``w``: q, q.b, k, k.b, v, v.b, talk, o,
    o.b.  Queries and keys are rotated, then divided by their root mean square."""
    T = x.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T, device=x.device)
    q = (x @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (x @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (x @ w["v"].T + w["v.b"]).view(T, G, vd)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rms(rotate_half(q, pos, int(rot["dims"]), float(rot["base"])), eps)
    k = rms(rotate_half(k, pos, int(rot["dims"]), float(rot["base"])), eps)
    out = pooled_rows(q, k, v, int(m["mask"]["size"]), int(m["mask"].get("pool") or 0), float(m["scale"]),
                      float(m.get("softcap") or 0.0), w["talk"])
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


def scan_rows(u, dt, A, B, C, D, S=None):
    """``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n``, ``y_c = sum_n S[c, n] C_n + D_c u_c``, token by
    token.  ``u``, ``dt`` [T, inner]; ``A`` [inner, N]; ``B``, ``C`` [T, N].  Returns (y [T, inner], the last S)."""
    T, inner = u.shape
    S = torch.zeros((inner, A.shape[1]), dtype=u.dtype, device=u.device) if S is None else S.clone()
    y = torch.zeros((T, inner), dtype=u.dtype, device=u.device)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y, S


def selective_scan(x, w, m: dict):
    """The state-space half of the ``parallel`` mixer on a whole sequence.  ``w``: in, conv, conv.b, x, dt, dt.b,
    A_log, D, o."""
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = x @ w["in"].T
    u, z = xz[:, :inner], xz[:, inner:]
    u = F.silu(causal_conv(u, w["conv"], w["conv.b"]))
    proj = u @ w["x"].T
    dt, B, C = proj[:, :R], proj[:, R: R + N], proj[:, R + N: R + 2 * N]
    dt = F.softplus(dt @ w["dt"].T + w["dt.b"])                              # [T, inner]
    y, _ = scan_rows(u, dt, -torch.exp(w["A_log"]), B, C, w["D"])
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


def forward(weights: dict, cfg: dict, tokens, return_layers: bool = False, chosen=None, want_routing: bool = False,
            compute=torch.float32):
    """Logits [T, vocab] of one whole sequence.  ``return_layers``: also the stream after every layer and the
    experts every routed layer chose.  ``want_routing``: also, per routed layer, (chosen [T, top], margin [T]: how
    far the last chosen expert's choice score lies above the first one not chosen).  ``chosen``: per routed layer,
    experts to take instead of choosing."""
    eps = float(cfg["norm"]["eps"])
    weights = {k: (v.to(compute) if v.is_floating_point() else v) for k, v in weights.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long, device=weights["embed"].device)
    x = weights["embed"][ids]
    v_first, layers, picks, routing, routed = None, [], [], [], 0
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
            y, idx, margin = routed_ff(x, sub(weights, p + "mlp."), layer["mlp"],
                                       None if chosen is None else chosen[routed])
            routed += 1
            picks.append(idx)
            routing.append((idx, margin))
            x = x + scalar_norm(y, weights[p + "norm2"], eps)
        layers.append(x.clone())
    logits = scalar_norm(x, weights["final.norm"], eps) @ weights["head"].T
    if return_layers:
        return logits, layers, picks
    return (logits, routing) if want_routing else logits


def generate(weights: dict, cfg: dict, prompt, max_new_tokens: int) -> list[int]:
    """Greedy continuation, the whole sequence recomputed for every token."""
    toks = list(prompt)
    for _ in range(max_new_tokens):
        toks.append(int(torch.argmax(forward(weights, cfg, toks)[-1])))
    return toks[len(prompt):]


def draw_weights(cfg: dict, seed: int, bias_rows: int = 10, matrix_dtype=torch.bfloat16) -> dict:
    """Random weights for a configuration, at scales where every mechanism matters: projections of unit gain with
    biases, distance biases and sinks as large as the scores' spread, blending fractions away from 0 and 1, head
    mixing away from the identity, step sizes and decays spread over a wide range, router corrections as large as
    the scores' differences.  Every tensor is rounded to ``matrix_dtype``."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    width, vocab = cfg["width"], cfg["vocab"]

    def put(name, t):
        W[name] = t.to(matrix_dtype)

    def mat(name, out, inn, gain=1.0):
        put(name, torch.randn(out, inn, generator=g) * gain / math.sqrt(inn))

    def vec(name, n, mean=0.0, spread=0.3):
        put(name, mean + spread * torch.randn(n, generator=g))

    def scalar(name, lo, hi):
        put(name, torch.tensor(lo + (hi - lo) * float(torch.rand((), generator=g))))

    def attention(p, m):
        Q, K, V = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        mat(p + "q", Q, width); mat(p + "k", K, width); mat(p + "v", V, width); mat(p + "o", width, m["heads"] * m["vdim"])
        vec(p + "q.b", Q); vec(p + "k.b", K); vec(p + "v.b", V); vec(p + "o.b", width)

    put("embed", torch.randn(vocab, width, generator=g))
    mat("head", vocab, width, 2.0)
    scalar("final.norm", 0.7, 1.4)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        scalar(p + "norm1", 0.5, 1.2)
        if layer["type"] == "attention":
            attention(p + "mix.", m)
            vec(p + "mix.rel", (int(m.get("bias_rows", bias_rows)), m["heads"]), spread=1.0)
            vec(p + "mix.sink", m["heads"], mean=0.5, spread=1.0)
            scalar(p + "mix.vmix", 0.25, 0.75)
        else:
            left, right = m["left"], m["right"]
            attention(p + "mix.left.", left)
            H = left["heads"]
            put(p + "mix.left.talk", 0.6 * torch.eye(H) + 0.4 * torch.randn(H, H, generator=g) / math.sqrt(H))
            C, N, R, taps = right["inner"], right["state"], right["dt_rank"], right["conv"]
            q = p + "mix.right."
            mat(q + "in", 2 * C, width); mat(q + "conv", C, taps, 1.5); vec(q + "conv.b", C)
            mat(q + "x", R + 2 * N, C); mat(q + "dt", C, R, 1.5); vec(q + "dt.b", C, mean=-1.0, spread=1.0)
            put(q + "A_log", torch.log(0.2 + 3.0 * torch.rand(C, N, generator=g)))
            vec(q + "D", C, mean=1.0); mat(q + "o", width, C)
        mlp = layer.get("mlp")
        if mlp is not None:
            scalar(p + "norm2", 0.5, 1.2)
            E, ident = int(mlp["router"]["experts"]), int(mlp["router"].get("identity") or 0)
            mat(p + "mlp.router", E + ident, width, 1.5)
            vec(p + "mlp.correction", E + ident, spread=0.05)
            names = [f"e{e}" for e in range(E)] + (["shared"] if mlp.get("shared") is not None else [])
            for n in names:
                ff = int(mlp["shared"]["ff"]) if n == "shared" else int(mlp["expert"]["ff"])
                mat(f"{p}mlp.{n}.gate", ff, width); mat(f"{p}mlp.{n}.up", ff, width); mat(f"{p}mlp.{n}.down", width, ff)
    return W
