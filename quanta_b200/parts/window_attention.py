"""Sliding-window grouped-query attention with extras, over the paged cache.

The core: ``q, k, v = W_q x, W_k x, W_v x`` (biases optional), q head ``h`` reads kv head ``h // (n_q / n_kv)``,
``score = (q . k) * scale`` over the last ``window`` keys of the request, softmax in float32, ``P V``, ``W_o``.
Each extra is a parameter and is off unless it is given:

* ``position``: a rotation of the first dims of every q / k head (the position parts); ``unit_qk``: every q and k
  head is divided by its root mean square over the head (no gains).  Rotating pairs leaves a head's mean square
  as it is, so the division commutes with the rotation; the kernel divides first.
* ``distance_bias=(rows, far)``: a learned table ``rel`` ``[rows, heads]`` whose row ``bucket(i - j)`` is added to
  the score (after the scale); the first ``rows // 2`` rows are the distances themselves, the rest a logarithmic
  ladder that reaches the last row at distance ``far``.  The table is spread over the distances below the window
  when the weights are loaded.
* ``sink``: one learned number per head whose exponential is one more term of the softmax denominator.
* ``softcap`` c: ``score <- c * tanh(score / c)``.
* ``pool`` P: beside the window, one key and one value per block of P tokens that lies wholly before the window
  (block b, positions ``bP .. bP + P - 1``, is read from position ``bP + P - 1 + window`` on): the means of the
  block's keys and values as the cache holds them.  They live in pages of their own with one row per P tokens.
* ``talk``: a learned ``[heads, heads]`` matrix that mixes the heads' softmax weights, ``w'_h = sum_g talk[h, g] w_g``;
  head h applies ``w'_h`` to the values of its own kv head.
* ``value_blend``: ``"source"``: the layer leaves its values (per token of the step, float32) under ``blend_key``
  for later layers; ``"blend"``: its values become ``(1 - lambda) v + lambda v_source`` with the learned number
  ``vmix`` before they are cached.  A source layer has no fraction of its own.

Scores, softmax weights, the bias, the sink and the mixing of heads are float32; the projections' float32
accumulators (with the biases) feed the kernel that norms, rotates and fills the cache.
"""

from __future__ import annotations

import math

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Addends, CacheSpec, CacheStream, KeepAll, Mixer, TensorSpec, Window, WindowAndOpenBlock, make, register


def distance_buckets(n_distances: int, rows: int, far: float) -> list[int]:
    """Row of the bias table for each distance ``0 .. n_distances - 1``."""
    half = rows // 2
    out = []
    for n in range(n_distances):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
            continue
        step = math.log(n / half) / math.log(far / half) * (rows - half)
        out.append(min(rows - 1, half + int(math.floor(step))))
    return out


@register("mixer", "window_attention")
class WindowAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int,
                 norm_eps: float, names: dict, value_dim: int | None = None, position=("none", {}),
                 unit_qk: bool = False, biases: bool = False, distance_bias: tuple | None = None, sink: bool = False,
                 softcap: float = 0.0, pool: int = 0, talk: bool = False, value_blend: str | None = None,
                 blend_key: str = "blend_values"):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} q heads are not a multiple of {n_kv_heads} kv heads")
        value_dim = head_dim if value_dim is None else int(value_dim)
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"head sizes {head_dim} / {value_dim}: the attention kernel takes 1 to 256")
        if window is None or int(window) < 1:
            raise ValueError(f"window {window}: a sliding window holds at least the token itself")
        if value_blend not in (None, "source", "blend"):
            raise ValueError(f"value_blend {value_blend!r} is not None, 'source' or 'blend'")
        if pool < 0 or softcap < 0:
            raise ValueError("pool and softcap cannot be negative (0: none)")
        self.hidden, self.nq, self.nkv, self.hd, self.vd = int(hidden_size), int(n_q_heads), int(n_kv_heads), int(head_dim), value_dim
        self.scale, self.window, self.eps = float(scale), int(window), float(norm_eps)
        self.unit_qk, self.biases, self.has_sink, self.has_talk = bool(unit_qk), bool(biases), bool(sink), bool(talk)
        self.softcap, self.pool = float(softcap), int(pool)
        self.distance_bias = None if distance_bias is None else (int(distance_bias[0]), float(distance_bias[1]))
        if self.distance_bias is not None and (self.distance_bias[0] < 1 or
                                               (self.distance_bias[0] > 1 and self.distance_bias[1] <= self.distance_bias[0] // 2)):
            raise ValueError(f"distance_bias {self.distance_bias}: the ladder must end beyond its first half")
        self.value_blend, self.blend_key = value_blend, blend_key
        self.position = make("position", position) if isinstance(position, tuple) else position
        self.names = dict(names)     # q, k, v, o (+ ".b" names q_b, k_b, v_b, o_b), rel, sink, talk, vmix
        self.w_qkv = self.w_o = self.b_qkv = self.b_o = self.dist_table = self.sink = self.talk = self.lam = None

    def children(self):
        return [self.position]

    def tensor_specs(self):
        n, W, hd, vd = self.names, self.hidden, self.hd, self.vd
        specs = [TensorSpec(n["q"], (self.nq * hd, W)), TensorSpec(n["k"], (self.nkv * hd, W)),
                 TensorSpec(n["v"], (self.nkv * vd, W)), TensorSpec(n["o"], (W, self.nq * vd))]
        if self.biases:
            specs += [TensorSpec(n["q_b"], (self.nq * hd,), "f32", "bias"), TensorSpec(n["k_b"], (self.nkv * hd,), "f32", "bias"),
                      TensorSpec(n["v_b"], (self.nkv * vd,), "f32", "bias"), TensorSpec(n["o_b"], (W,), "f32", "bias")]
        if self.distance_bias is not None:
            specs.append(TensorSpec(n["rel"], (self.distance_bias[0], self.nq), "f32", "bias"))
        if self.value_blend == "blend":
            specs.append(TensorSpec(n["vmix"], (), "f32", "fraction"))
        if self.has_sink:
            specs.append(TensorSpec(n["sink"], (self.nq,), "f32", "bias"))
        if self.has_talk:
            specs.append(TensorSpec(n["talk"], (self.nq, self.nq), "f32", "mixing"))
        return specs

    def load(self, fetch):
        n = self.names
        q = fetch(n["q"])
        a = self.nq * self.hd
        b = a + self.nkv * self.hd
        c = b + self.nkv * self.vd
        # one fused input projection, its rows padded to a multiple of 8 (every product row starts on 16 bytes)
        rows = -(-c // 8) * 8
        self.w_qkv = torch.zeros((rows, self.hidden), dtype=q.dtype, device=q.device)
        self.w_qkv[:a].copy_(q)
        del q
        self.w_qkv[a:b].copy_(fetch(n["k"]))
        self.w_qkv[b:c].copy_(fetch(n["v"]))
        self.w_o = fetch(n["o"])
        if self.biases:
            self.b_qkv = torch.cat([fetch(n["q_b"]), fetch(n["k_b"]), fetch(n["v_b"])]).contiguous()
            self.b_o = fetch(n["o_b"]).contiguous()
        if self.distance_bias is not None:
            rel = fetch(n["rel"])
            rows_of = distance_buckets(self.window, *self.distance_bias)
            self.dist_table = rel[torch.tensor(rows_of, dtype=torch.long, device=rel.device)].contiguous()
        if self.value_blend == "blend":
            self.lam = fetch(n["vmix"]).reshape(1).contiguous()
        if self.has_sink:
            self.sink = fetch(n["sink"]).contiguous()
        if self.has_talk:
            self.talk = fetch(n["talk"]).contiguous()

    def cache_spec(self):
        tokens = (CacheStream("k", self.nkv, self.hd), CacheStream("v", self.nkv, self.vd))
        if not self.pool:
            return CacheSpec(tokens, Window(self.window))
        # the tokens of a block stay until the block is whole (its means are taken from the pages); the means stay
        return (CacheSpec(tokens, WindowAndOpenBlock(self.window, self.pool)),
                CacheSpec((CacheStream("k_pooled", self.nkv, self.hd), CacheStream("v_pooled", self.nkv, self.vd)),
                          KeepAll(), stride=self.pool))

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        if cache is None or not cache.write:
            raise ValueError("window_attention fills a cache of its own")
        qkv = linear(x, self.w_qkv, out_dtype=torch.float32)
        q = torch.empty((T, self.nq, self.hd), dtype=x.dtype, device=x.device)
        tables = self.position.rotary_tables(x.device)
        if tables is None:
            inv_freq, pair_axis, rd = torch.empty(0, dtype=torch.float32, device=x.device), None, 0
        else:
            inv_freq, pair_axis, rd, _ = tables
        v_first = v_export = None
        if self.value_blend == "source":
            v_export = torch.empty((T, self.nkv * self.vd), dtype=torch.float32, device=x.device)
            ctx.work[self.blend_key] = v_export
        elif self.value_blend == "blend":
            v_first = ctx.work.get(self.blend_key)
            if v_first is None or v_first.shape != (T, self.nkv * self.vd):
                raise ValueError("window_attention: no earlier layer left values of this layer's size to blend with")
        kernels.qknorm_rope_write(
            qkv, q, cache.k, cache.v, None, None, kernels.NORM_PER_HEAD if self.unit_qk else kernels.NORM_NONE, self.eps,
            inv_freq, pair_axis, ctx.positions, ctx.tok_pos, ctx.tok_req, cache.tables["k"], self.nq, self.nkv, self.hd,
            rd, cache.page_size, ctx.status, vd=self.vd, bias=self.b_qkv, v_first=v_first, v_lambda=self.lam,
            v_export=v_export)
        pooled = {}
        if self.pool:
            kp, vp = cache.streams["k_pooled"], cache.streams["v_pooled"]
            kernels.pool_blocks(cache.k, cache.v, kp, vp, ctx.tok_pos, ctx.tok_req, cache.tables["k"],
                                cache.tables["k_pooled"], self.pool, ctx.status)
            pooled = dict(pool=self.pool, pooled_k=kp, pooled_v=vp, pool_table=cache.tables["k_pooled"])
        out = empty_rows(T, self.nq, self.vd, dtype=x.dtype, device=x.device)
        scratch = None
        if self.has_talk:
            scratch = torch.empty((T, self.nq, self.nkv, self.vd), dtype=torch.float32, device=x.device)
        kernels.window_attention(q, cache.k, cache.v, out, ctx.tok_pos, ctx.tok_req, cache.tables["k"], self.scale,
                                 self.window, ctx.status, dist_bias=self.dist_table, sink=self.sink,
                                 softcap=self.softcap, talk=self.talk, scratch=scratch,
                                 n_requests=int(ctx.req_start.numel()) - 1, **pooled)
        y = linear(out.view(T, self.nq * self.vd), self.w_o, out_dtype=torch.float32)
        return Addends(y, bias=self.b_o) if self.biases else y
