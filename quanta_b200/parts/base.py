"""What a part is, and the registries parts are chosen from.

A model is put together from parts of eight kinds: ``mixer`` (attention, or a recurrence with a state
of fixed size), ``feed_forward`` (dense or routed experts), ``norm``, ``position`` (position encoding),
``time_conv`` (a short convolution over time in front of a sublayer), ``block`` (how a layer arranges
the others), ``embedding`` (token ids to the residual stream) and ``head`` (the residual stream to
logits).  A part takes every size and constant as a constructor parameter, names
the checkpoint tensors it needs (``tensor_specs``), receives them (``load``) and runs on the tokens
of one step (``forward``).  No part knows which model it is in; an architecture is a function from
its configuration to a ``ModelSpec`` that names parts and parameters layer by layer.

Registering a new part: ``@register("mixer", "my_mixer") class MyMixer(Mixer): ...`` in any module
that is imported before the model is built.  The framework's files do not change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

KINDS = ("mixer", "feed_forward", "norm", "position", "time_conv", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {k: {} for k in KINDS}


def register(kind: str, name: str) -> Callable[[type], type]:
    if kind not in _REGISTRY:
        raise KeyError(f"unknown part kind {kind!r}; kinds: {KINDS}")

    def deco(cls: type) -> type:
        _REGISTRY[kind][name] = cls
        return cls

    return deco


def registered(kind: str) -> list[str]:
    return sorted(_REGISTRY[kind])


def make(kind: str, choice) -> Any:
    """Instantiate ``(name, params)`` of the given kind."""
    name, params = choice
    try:
        cls = _REGISTRY[kind][name]
    except KeyError:
        raise KeyError(f"no {kind} part named {name!r}; registered: {registered(kind)}") from None
    return cls(**params)


# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part needs.

    ``kind``: ``"matrix"`` is held in the model's compute dtype (bfloat16 or float32); ``"f32"`` is
    held in float32 whatever the compute dtype (norm gains, router gate and bias: a tensor stored in
    32-bit stays so); ``"i32"`` integer tables.  ``init`` tells the random-weights mode how to draw
    it: ``"normal"`` N(0, 0.02), ``"gain"`` 1 + U(-0.1, 0.1), ``"bias"`` U(-0.05, 0.05), ``"mixing"`` a square matrix, the
    identity + U(-0.1, 0.1), ``"fraction"`` U(0.2, 0.8), ``"depth_mix"`` a vector U(-0.3, 0.3) whose last entry has 1 added, ``"conv"`` taps U(-0.4, 0.4) with 1 added to the newest.
    """
    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class CacheStream:
    """One paged tensor a mixer keeps per token: ``heads`` rows of ``width`` elements in the activation
    dtype.  Softmax attention keeps two (keys and values); a mixer that attends over one latent vector
    keeps one; widths need not be equal."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class Retention:
    """Which cached positions a request's future queries can still read.  The cache manager gives a
    page back as soon as no position of it is needed any more, and never asks again about a page it
    gave back, so what is needed may only shrink as the request grows.  The base keeps everything."""

    def needed_ranges(self, length: int) -> list[tuple[int, int | None]]:
        """Half-open position ranges ``(lo, hi)`` that queries at positions ``>= length`` may read, given
        that ``length`` tokens are cached; ``hi`` None: no upper end.  The last range must be open."""
        return [(0, None)]


@dataclass(frozen=True)
class KeepAll(Retention):
    pass


@dataclass(frozen=True)
class Window(Retention):
    """A query at position p reads the keys ``p - window + 1 .. p`` only."""
    window: int = 1

    def needed_ranges(self, length):
        return [(max(0, length - self.window + 1), None)]


@dataclass(frozen=True)
class WindowAndOpenBlock(Retention):
    """A window, and besides the tokens of the block of ``block`` tokens that is not whole yet (a mixer that
    summarises every whole block from the pages reads them once more when the block's last token arrives)."""
    window: int = 1
    block: int = 1

    def needed_ranges(self, length):
        return [(max(0, min(length - self.window + 1, length // self.block * self.block)), None)]


@dataclass(frozen=True)
class CacheSpec:
    """A mixer's need of paged per-token storage: its streams and what is retained.  Layers with equal
    specs form one group of the cache manager: they share pages ids and block tables.  ``stride`` > 1: the
    streams hold one row per ``stride`` tokens (row ``p // stride`` belongs to position ``p``: a summary of
    every block of that many tokens), so a page of ``page_size`` rows covers ``page_size * stride`` positions;
    the retention rule still speaks of token positions.  A mixer that keeps rows per token and rows per block
    declares two specs (``Mixer.cache_spec`` may return a tuple); every stream of a mixer has its own name."""
    streams: tuple[CacheStream, ...]
    retention: Retention = KeepAll()
    stride: int = 1

    @property
    def window(self) -> int | None:
        return getattr(self.retention, "window", None)


def KVCacheSpec(n_kv_heads: int, head_dim: int, window: int | None = None) -> CacheSpec:
    """Keys and values of softmax attention: two streams of ``n_kv_heads`` x ``head_dim``; ``window`` None:
    all keys are kept, W: only the last W positions."""
    return CacheSpec((CacheStream("k", n_kv_heads, head_dim), CacheStream("v", n_kv_heads, head_dim)),
                     KeepAll() if window is None else Window(int(window)))


class LayerCache:
    """What a mixer sees of the cache in one step: its own pages of every stream it declared
    (``streams[name]`` ``[num_pages, heads, page_size, width]``) and its group's block table (int32
    ``[requests in the step, pages per request]``, -1 where a page was given back).  ``write`` False:
    this layer reads a cache another layer wrote.  ``k`` / ``v`` are the streams of those names.  A mixer
    with several cache specs finds the block table of each stream's group in ``tables[name]``
    (``block_table`` is the first spec's)."""

    def __init__(self, k=None, v=None, page_size: int = 0, block_table=None, write: bool = True, streams=None,
                 tables=None):
        self.streams = dict(streams) if streams is not None else {"k": k, "v": v}
        self.page_size, self.block_table, self.write = page_size, block_table, write
        self.tables = dict(tables) if tables is not None else {name: block_table for name in self.streams}

    @property
    def k(self):
        return self.streams["k"]

    @property
    def v(self):
        return self.streams["v"]


@dataclass
class StepContext:
    """Per-step facts every part may read.  All tensors are on the device; ``T`` tokens in the step.

    The tokens of request row ``r`` are the rows ``req_start[r] .. req_start[r+1]`` of every activation,
    in position order; its per-request state (a mixer's ``state_spec``) is row ``req_slot[r]`` of each
    state tensor.  A part that reads only these device arrays (no ``host``, no ``.item()``) may declare
    itself ``graph_safe``; one part that is not turns captured decode steps off for the whole model.
    ``positions`` carries one coordinate per position axis; the step function feeds every axis the
    token's text position (a caller cannot hand a token several coordinates: image inputs are not built)."""
    n_tokens: int
    positions: torch.Tensor            # int32 [T, axes]   position fed to the position encoding
    tok_pos: torch.Tensor              # int32 [T]         index of the token in its request's cache
    tok_req: torch.Tensor              # int32 [T]         row of the token's request in this step
    req_slot: torch.Tensor             # int32 [R]         state slot of each request of the step
    req_start: torch.Tensor            # int32 [R+1]       first token row of each request
    req_len_after: torch.Tensor        # int32 [R]         tokens cached once the step is done
    status: torch.Tensor               # int32 [4]         device error words
    dtype: torch.dtype                 # activation dtype
    max_new_tokens_per_req: int = 0    # largest portion in the step
    max_len_after: int = 0             # largest req_len_after (host copy, for launch sizing)
    host: dict = field(default_factory=dict)   # host copies of the small arrays, for parts that need them
    # how the step's tokens fall into requests, for mixers that treat single tokens and portions
    # differently: rows of requests that bring exactly one token, and (request row, first token row,
    # tokens) of the others.  None: derived from host["req_start"], or one portion holding everything.
    dec_tok: torch.Tensor | None = None        # int32 [n_dec] token rows (device)
    n_dec: int = 0
    spans: list | None = None
    work: dict = field(default_factory=dict)   # per-step scratch shared by the layers (tile lists and the like)


class Part:
    """Base of every part."""

    # True when ``forward`` reads nothing from the host (no ``ctx.host``, no ``.item()``, no shapes that
    # depend on data): a decode step of such parts can be captured in a CUDA graph and replayed.
    graph_safe = False

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, fetch: Callable[[str], torch.Tensor]) -> None:
        """Receive the tensors named in ``tensor_specs``: ``fetch(name)`` returns the device tensor in
        the dtype its kind asks for."""

    def children(self) -> list["Part"]:
        return []


_SIDE_STREAMS: dict = {}          # device index -> the second stream of that device


def run_beside(side_fn, main_fn, device):
    """Two pieces of work that share nothing but their inputs, ``side_fn()`` on a second CUDA stream beside
    ``main_fn()`` on the current one; returns ``(side result, main result)``.  The streams fork and join inside the
    launch order (the second stream waits for everything launched so far, the current one then waits for it), also in
    a captured step; what the side work allocates is used afterwards on the current stream only behind that join, and
    the next fork comes behind the current stream's use of it.  Not on a CUDA device: one after the other."""
    if torch.device(device).type != "cuda":
        return side_fn(), main_fn()
    dev = torch.device(device)
    main = torch.cuda.current_stream(dev)
    side = _SIDE_STREAMS.get(dev.index)
    if side is None:
        side = _SIDE_STREAMS[dev.index] = torch.cuda.Stream(device=dev)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        b = side_fn()
    a = main_fn()
    main.wait_stream(side)
    return b, a


class Addends:
    """A sublayer's output as a sum that nobody has taken yet:
    ``scale * n_y(sum_s y[:, s] + bias) + extra_scale * n_e(extra + extra_bias)`` with ``y`` float32 ``[T, H]`` or
    ``[T, S, H]``, ``extra`` float32 ``[T, H]`` or None and biases of ``H`` numbers or None.  ``n_y`` / ``n_e`` are the
    identity, or with ``y_gain`` / ``extra_gain`` (float32 ``[H]``) an RMS norm of the addend over the whole row with
    that gain (``branch_eps`` inside the root): two branches that are each normed before they are summed.  A mixer or
    feed-forward whose block norms its output may return one instead of a tensor: the norm kernel that reads the
    output takes the sum in the same launch (an output bias, two branches with a weight each, routed slots and a
    shared expert)."""

    def __init__(self, y, scale: float = 1.0, bias=None, extra=None, extra_scale: float = 1.0, extra_bias=None,
                 y_gain=None, extra_gain=None, branch_eps: float = 0.0):
        self.y, self.scale, self.bias = y, float(scale), bias
        self.extra, self.extra_scale, self.extra_bias = extra, float(extra_scale), extra_bias
        self.y_gain, self.extra_gain, self.branch_eps = y_gain, extra_gain, float(branch_eps)

    @property
    def branch_normed(self) -> bool:
        return self.y_gain is not None or self.extra_gain is not None

    def total(self) -> torch.Tensor:
        """The sum as a float32 ``[T, H]`` tensor (plain torch; for tools, not for the step)."""
        def normed(z, gain):
            if gain is None:
                return z
            return gain * z * torch.rsqrt((z * z).mean(-1, keepdim=True) + self.branch_eps)

        y = self.y.float()
        z = y.sum(1) if y.dim() == 3 else y.clone()
        if self.bias is not None:
            z += self.bias
        z = normed(z, self.y_gain) * self.scale
        if self.extra is not None:
            e = self.extra.float() + (self.extra_bias if self.extra_bias is not None else 0.0)
            z += self.extra_scale * normed(e, self.extra_gain)
        return z


class NormedPending:
    """A pending contribution that is normed before it joins the residual stream: ``y`` (float32 ``[T, H]``, a
    sublayer's output, or an ``Addends`` whose sum is that output) and the norm part that is applied to it.  A norm
    that gets one as its ``delta`` norms ``y``, adds it and norms the sum in one launch when it can
    (``Norm.forward`` of the built-in norms); whoever needs the plain numbers calls ``materialize``."""

    def __init__(self, y, norm: "Norm"):
        if isinstance(y, Addends):
            self.addends = y
        else:
            self.addends = Addends(y if y.dtype == torch.float32 else y.float())
        self.norm = norm

    @property
    def y(self) -> torch.Tensor:
        a = self.addends
        plain = a.y.dim() == 2 and a.scale == 1.0 and a.bias is None and a.extra is None and not a.branch_normed
        return a.y if plain else a.total()

    def materialize(self) -> torch.Tensor:
        y = self.y
        d = torch.empty(y.shape, dtype=torch.float32, device=y.device)
        self.norm.forward(y, None, d)
        return d


class StreamCopy:
    """Nothing is pending, and the residual stream as it stands is already at hand in the activation dtype (``x``
    ``[T, H]``, laid out by ``matmul.empty_rows``): whoever finished the stream wrote the copy in the same launch, so
    a sublayer that reads the stream without a norm needs no launch of its own to get it."""

    def __init__(self, x: torch.Tensor):
        self.x = x


class StreamsPending:
    """A pending contribution of a model that keeps several residual streams ``x_1 .. x_S``: the sublayer's output
    ``y`` (``[T, H]``, or ``[T, K, H]`` partial results that are added in order) and how it is written back,
    ``x_t <- sum_s mix[s, t] x_s + mult * out_w[t] * y`` for all streams at once.  The norm that reads the streams
    next does the write-back in its own launch (``Norm.forward_streams``; a plain ``forward`` of the built-in
    norm reads the sum of the streams, which is what the output head wants)."""

    def __init__(self, y: torch.Tensor, mix: torch.Tensor, out_w: torch.Tensor, mult: float):
        self.y, self.mix, self.out_w, self.mult = y, mix, out_w, float(mult)


class Norm(Part):
    def forward(self, h: torch.Tensor, delta, out, rows=None, store_h=True) -> None:
        """``delta``: None, a tensor ``[T, H]`` / ``[T, S, H]``, a ``NormedPending``, or (with ``h`` the streams
        ``[T, S, H]`` of a model that keeps several) a ``StreamsPending``."""
        raise NotImplementedError

    def forward_streams(self, x: torch.Tensor, pending, read_w, out, rows=None, store=True) -> None:
        """Several residual streams ``x`` ``[T, S, H]``: write ``pending`` (a ``StreamsPending`` or None) back,
        read ``u = sum_t read_w[t] x_t`` (``read_w`` None: the plain sum) and norm ``u`` into ``out``."""
        raise NotImplementedError(f"{type(self).__name__} does not read several residual streams")


class PositionEncoding(Part):
    """Turns positions into what a mixer consumes.  ``rotary_tables`` returns ``(inv_freq float32
    [rd/2], pair_axis int32 [rd/2] or None, rotary_dim, n_axes)`` or None when nothing is rotated."""

    n_axes = 1

    def rotary_tables(self, device):
        return None


class Mixer(Part):
    def cache_spec(self) -> CacheSpec | tuple[CacheSpec, ...] | None:
        """What the mixer keeps per token in pages (streams and retention); None: nothing.  A tuple: several
        needs with different retention or stride, each a page group of its own."""
        return None

    def state_spec(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        """Per-request state of fixed size: name -> (shape, dtype).  The cache manager keeps one row per
        state slot, zeroed when a request takes the slot."""
        return {}

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache | None,
                state: dict[str, torch.Tensor]) -> torch.Tensor:
        """``x`` [T, hidden] in the activation dtype -> the layer's contribution to the residual stream,
        [T, hidden] or [T, S, hidden] (S partial results the next norm sums in order)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class TimeConv(Part):
    """A short causal convolution over a request's rows.  Its last inputs are per-request state:
    ``state_spec`` names them like a mixer's, and ``forward(x float32 [T, C], ctx, state, out)`` reads and
    updates the rows ``ctx.req_slot`` of ``state[name]``."""

    def state_spec(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        return {}

    def forward(self, x: torch.Tensor, ctx: StepContext, state: dict[str, torch.Tensor], out: torch.Tensor) -> None:
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the float32 residual stream: ``forward(ids int32 [T], ctx) -> [T, hidden]``."""

    def forward(self, ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """The residual stream to logits: ``forward(h, pending, rows, ctx)`` adds the last layer's pending
    contribution for the wanted token rows ``rows`` (int32) and returns float32 ``[len(rows), vocab]``."""

    def forward(self, h: torch.Tensor, pending, rows: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of norm, mixer and feed-forward in one layer.  ``forward`` takes the residual stream
    ``h`` (float32) and the not-yet-added contribution of the layer before, and returns the new pending
    contribution; every addition to ``h`` happens inside a norm kernel."""

    def state_spec(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        """Per-request state of the whole layer: the mixer's, plus what the block's other parts keep."""
        return self.mixer.state_spec()

    def forward(self, h, pending, ctx, cache, state):
        raise NotImplementedError
