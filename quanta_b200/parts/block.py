"""Layer arrangement, embedding and output head.

Pre-norm block with two residual sums (src/quanta/minimax/model.py:70-73):
``h = h + mixer(norm_1(h)); h = h + feed_forward(norm_2(h))``.  The sums are taken in float32 inside
the norm kernels: a part's output stays "pending" until the next norm reads the row.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from . import norms as _norms
from .base import Addends, Block, Embedding, Head, NormedPending, StreamCopy, StreamsPending, TensorSpec, make, register


@register("block", "pre_norm")
class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, hidden_size: int, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.hidden = int(hidden_size)
        self.mixer = make("mixer", mixer)
        self.feed_forward = make("feed_forward", feed_forward)
        self.mixer_norm = make("norm", mixer_norm)
        self.feed_forward_norm = make("norm", feed_forward_norm)

    def children(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, h, pending, ctx, cache, state):
        x = empty_rows(h.shape[0], self.hidden, dtype=ctx.dtype, device=h.device)
        self.mixer_norm.forward(h, pending, x)
        a = self.mixer.forward(x, ctx, cache, state)
        x2 = empty_rows(h.shape[0], self.hidden, dtype=ctx.dtype, device=h.device)
        self.feed_forward_norm.forward(h, a, x2)
        return self.feed_forward.forward(x2, ctx)


@register("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after each sublayer: ``h += post_1(mixer(conv(pre_1(h))))`` and, where the
    layer has a feed-forward, ``h += post_2(feed_forward(pre_2(h)))``.  ``conv`` (optional) is a short
    convolution over time on the mixer's input; its last inputs are part of the layer's per-request state.
    Both sums are float32 and happen inside the next pre-norm (or the head's norm), which also applies the
    post-norm to the sublayer's float32 output: a contribution is never rounded to the activation dtype."""

    graph_safe = True

    def __init__(self, hidden_size: int, mixer, mixer_norm, mixer_post_norm, feed_forward=None,
                 feed_forward_norm=None, feed_forward_post_norm=None, conv=None):
        self.hidden = int(hidden_size)
        self.mixer = make("mixer", mixer)
        self.mixer_norm = make("norm", mixer_norm)
        self.mixer_post_norm = make("norm", mixer_post_norm)
        self.conv = make("time_conv", conv) if conv is not None else None
        self.feed_forward = make("feed_forward", feed_forward) if feed_forward is not None else None
        self.feed_forward_norm = self.feed_forward_post_norm = None
        if self.feed_forward is not None:
            self.feed_forward_norm = make("norm", feed_forward_norm)
            self.feed_forward_post_norm = make("norm", feed_forward_post_norm)

    def children(self):
        parts = [self.mixer_norm, self.conv, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                 self.feed_forward, self.feed_forward_post_norm]
        return [p for p in parts if p is not None]

    def state_spec(self):
        spec = dict(self.mixer.state_spec())
        if self.conv is not None:
            for name, need in self.conv.state_spec().items():
                if name in spec:
                    raise ValueError(f"the mixer and the convolution both keep a state named {name!r}")
                spec[name] = need
        return spec

    def forward(self, h, pending, ctx, cache, state):
        T = h.shape[0]
        if isinstance(pending, StreamCopy):
            # the stream is finished and its copy in the activation dtype came with it
            ready, pending = pending.x, None
            if self.conv is None and isinstance(self.mixer_norm, _norms.NoNorm) and ready.dtype == ctx.dtype:
                x = ready
            else:
                ready = None
        else:
            ready = None
        if ready is None:
            x = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device)
        if ready is not None:
            pass
        elif self.conv is None:
            self.mixer_norm.forward(h, pending, x)
        else:
            normed = torch.empty((T, self.hidden), dtype=torch.float32, device=h.device)
            self.mixer_norm.forward(h, pending, normed)
            self.conv.forward(normed, ctx, state, x)
        # a sublayer's output stays pending together with its post-norm: the next pre-norm (or the head's norm)
        # norms it, adds it to the stream and norms the sum in one launch
        d = NormedPending(self.mixer.forward(x, ctx, cache, state), self.mixer_post_norm)
        if self.feed_forward is None:
            return d
        x2 = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device)
        self.feed_forward_norm.forward(h, d, x2)
        return NormedPending(self.feed_forward.forward(x2, ctx), self.feed_forward_post_norm)


@register("block", "hyper_connected")
class HyperConnectedBlock(Block):
    """Pre-norm sublayers over ``streams`` copies ``x_1 .. x_S`` of the residual stream.  Sublayer q (the mixer,
    then the feed-forward where the layer has one) reads ``u = sum_s in_q[s] x_s``, computes
    ``y = sublayer(norm_q(u))`` and writes back ``x_t <- sum_s mix_q[s, t] x_s + mult * out_q[t] * y`` for all
    streams at once (``mix_q`` is indexed ``[from, to]``).  ``names`` gives the tensors ``in1, mix1, out1, in2,
    mix2, out2``; None: unit weights and the identity, which with one stream is the usual pre-norm residual
    ``x += mult * sublayer(norm(x))``.  Streams, sums and norms are float32; the write-back of a sublayer, the
    read of the next and its norm are one launch (the model's head reads the sum of the streams the same way)."""

    graph_safe = True

    def __init__(self, hidden_size: int, streams: int, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None,
                 residual_mult: float = 1.0, names: dict | None = None):
        if not 1 <= int(streams) <= kernels.MAX_STREAMS:
            raise ValueError(f"{streams} residual streams: the kernel takes 1 to {kernels.MAX_STREAMS}")
        self.hidden, self.S, self.mult = int(hidden_size), int(streams), float(residual_mult)
        self.mixer = make("mixer", mixer)
        self.mixer_norm = make("norm", mixer_norm)
        self.feed_forward = make("feed_forward", feed_forward) if feed_forward is not None else None
        self.feed_forward_norm = make("norm", feed_forward_norm) if feed_forward is not None else None
        self.names = dict(names) if names is not None else None
        self.w: dict[str, torch.Tensor] = {}

    def _sublayers(self):
        return ("1", "2") if self.feed_forward is not None else ("1",)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        if self.names is None:
            return []
        specs = []
        for q in self._sublayers():
            specs += [TensorSpec(self.names["in" + q], (self.S,), "f32", "gain"),
                      TensorSpec(self.names["mix" + q], (self.S, self.S), "f32", "mixing"),
                      TensorSpec(self.names["out" + q], (self.S,), "f32", "gain")]
        return specs

    def load(self, fetch):
        if self.names is not None:
            for q in self._sublayers():
                for k in ("in", "mix", "out"):
                    self.w[k + q] = fetch(self.names[k + q]).contiguous()

    def _weights(self, device):
        if not self.w:
            for q in self._sublayers():
                self.w["in" + q] = torch.ones(self.S, dtype=torch.float32, device=device)
                self.w["mix" + q] = torch.eye(self.S, dtype=torch.float32, device=device)
                self.w["out" + q] = torch.ones(self.S, dtype=torch.float32, device=device)
        return self.w

    def forward(self, h, pending, ctx, cache, state):
        x = h if h.dim() == 3 else h.unsqueeze(1)
        if x.shape[1] != self.S:
            raise ValueError(f"the layer is connected to {self.S} residual streams; the model keeps {x.shape[1]}")
        w = self._weights(h.device)
        T = x.shape[0]
        u = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device)
        self.mixer_norm.forward_streams(x, pending, w["in1"], u)
        d = StreamsPending(self.mixer.forward(u, ctx, cache, state), w["mix1"], w["out1"], self.mult)
        if self.feed_forward is None:
            return d
        u2 = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device)
        self.feed_forward_norm.forward_streams(x, d, w["in2"], u2)
        return StreamsPending(self.feed_forward.forward(u2, ctx), w["mix2"], w["out2"], self.mult)


@register("block", "depth_weighted")
class DepthWeightedBlock(Block):
    """Any single-stream block, after which the residual stream is replaced by a learned weighted sum of the results
    so far: with ``X_0`` the stream the first such layer starts from and ``X_(i+1)`` the result of layer ``i`` (the
    inner block's whole effect on the stream it was given), the stream that goes on is
    ``sum_{j <= i+1} weights[j] * X_j``.  ``index`` is ``i``; ``weights_name`` names a float32 tensor of ``i + 2``
    numbers.  The results of the step's tokens are kept in one float32 tensor ``[depth + 1, T, hidden]`` that the
    layers of a step share (``ctx.work``); the inner block's last contribution joins the stream, the result is
    stored and the weighted sum is taken in ONE launch."""

    def __init__(self, hidden_size: int, inner, index: int, depth: int, weights_name: str, history_key: str = "depth_results"):
        if not 0 <= int(index) < int(depth):
            raise ValueError(f"depth_weighted: layer {index} of {depth}")
        self.hidden, self.index, self.depth = int(hidden_size), int(index), int(depth)
        self.inner = make("block", inner)
        self.weights_name, self.history_key = weights_name, history_key
        self.weights = None
        self.graph_safe = bool(getattr(self.inner, "graph_safe", False))

    # the model asks a block for its mixer and feed-forward (cache needs, routing traces)
    @property
    def mixer(self):
        return self.inner.mixer

    @property
    def feed_forward(self):
        return getattr(self.inner, "feed_forward", None)

    def children(self):
        return [self.inner]

    def state_spec(self):
        return self.inner.state_spec()

    def tensor_specs(self):
        return [TensorSpec(self.weights_name, (self.index + 2,), "f32", "depth_mix")]

    def load(self, fetch):
        self.weights = fetch(self.weights_name).contiguous()

    def forward(self, h, pending, ctx, cache, state):
        if h.dim() != 2:
            raise NotImplementedError("a depth-weighted stream is built for one residual stream")
        ready = None
        if isinstance(pending, StreamCopy):
            ready, pending = pending, None
        if pending is not None:
            raise ValueError("a depth-weighted layer starts from a finished stream (nothing pending)")
        T = h.shape[0]
        hist = ctx.work.get(self.history_key)
        if self.index == 0 or hist is None:
            if self.index != 0:
                raise ValueError("depth_weighted: the results of the earlier layers of this step are missing")
            hist = ctx.work[self.history_key] = torch.empty((self.depth + 1, T, self.hidden), dtype=torch.float32,
                                                            device=h.device)
            hist[0].copy_(h)
        d = self.inner.forward(h, ready, ctx, cache, state)
        # the next layer of the stack reads the stream it is given: its copy in the activation dtype is written here
        out = empty_rows(T, self.hidden, dtype=ctx.dtype, device=h.device) if self.index + 1 < self.depth else None
        if isinstance(d, NormedPending) and isinstance(d.norm, _norms.RMSNorm):
            _norms.normed_add(h, d, None, 0.0, out, None, True, history=hist, n_history=self.index + 1,
                              history_weights=self.weights)
            return StreamCopy(out) if out is not None else None
        if isinstance(d, (NormedPending, Addends)):
            d = d.materialize() if isinstance(d, NormedPending) else d.total()
        if isinstance(d, StreamsPending):
            raise NotImplementedError("a depth-weighted stream is built for one residual stream")
        if d is not None and d.dtype != torch.float32:
            d = d.float()
        kernels.grouped_normed_add(h, y=d, history=hist, n_history=self.index + 1, history_weights=self.weights, out=out)
        return StreamCopy(out) if out is not None else None


@register("embedding", "token_table")
class TokenTable(Embedding):
    """``h = table[ids] * scale`` into the float32 residual stream (src/quanta/minimax/model.py:91; the
    reference has no scale).  ``positions_name``: a second table ``[max_positions, hidden]`` whose row of the
    token's position is added (not scaled).  ``streams`` > 1: the model keeps that many residual streams, which
    all start as this row (``[T, streams, hidden]``)."""

    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str, scale: float = 1.0,
                 positions_name: str | None = None, max_positions: int = 0, streams: int = 1):
        self.V, self.H, self.weight_name, self.scale = int(vocab_size), int(hidden_size), weight_name, float(scale)
        self.positions_name, self.max_positions, self.streams = positions_name, int(max_positions), int(streams)
        if positions_name is not None and self.max_positions <= 0:
            raise ValueError("a table of learned positions needs max_positions")
        self.table = self.pos_table = None

    def tensor_specs(self):
        specs = [TensorSpec(self.weight_name, (self.V, self.H))]
        if self.positions_name is not None:
            specs.append(TensorSpec(self.positions_name, (self.max_positions, self.H)))
        return specs

    def load(self, fetch):
        self.table = fetch(self.weight_name)
        if self.positions_name is not None:
            self.pos_table = fetch(self.positions_name)

    def forward(self, ids, ctx):
        shape = (ids.numel(), self.H) if self.streams == 1 else (ids.numel(), self.streams, self.H)
        if self.pos_table is not None and ctx.host and ctx.max_len_after > self.max_positions:
            raise ValueError(f"a request of {ctx.max_len_after} tokens: the model has learned positions for "
                             f"{self.max_positions}")
        h = torch.empty(shape, dtype=torch.float32, device=ids.device)
        kernels.embedding(h, self.table, ids, ctx.status, self.scale, self.pos_table, ctx.tok_pos)
        return h


@register("head", "linear")
class LinearHead(Head):
    """Final norm on the wanted rows, then ``logits = x @ head.T`` in float32
    (src/quanta/minimax/runtime.py:95-98).  ``tied_to`` names the embedding table to reuse (a tensor that
    two parts ask for by the same name is loaded once and shared); ``logit_scale`` multiplies the logits;
    ``softcap`` > 0: ``logits <- softcap * tanh(logits / softcap)`` at the end."""

    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, norm, weight_name: str | None, tied_to: str | None,
                 logit_scale: float = 1.0, softcap: float = 0.0):
        self.V, self.H, self.logit_scale = int(vocab_size), int(hidden_size), float(logit_scale)
        self.softcap = float(softcap)
        if self.softcap < 0:
            raise ValueError(f"linear head: a cap of {softcap} on the logits")
        self.norm = make("norm", norm)
        self.weight_name, self.tied_to = weight_name, tied_to
        self.weight = None

    def children(self):
        return [self.norm]

    def tensor_specs(self):
        return [TensorSpec(self.tied_to if self.tied_to else self.weight_name, (self.V, self.H))]

    def load(self, fetch):
        self.weight = fetch(self.tied_to if self.tied_to else self.weight_name)

    def forward(self, h, pending, rows, ctx):
        n = rows.numel()
        x = empty_rows(n, self.H, dtype=ctx.dtype, device=h.device)
        self.norm.forward(h, pending, x, rows=rows, store_h=False)
        logits = linear(x, self.weight, out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            logits.mul_(self.logit_scale)       # on the float32 products: one rounding, as the formula has it
        if self.softcap > 0.0:
            if not logits.is_contiguous():
                logits = logits.contiguous()
            kernels.tanh_cap(logits, self.softcap)
        return logits
