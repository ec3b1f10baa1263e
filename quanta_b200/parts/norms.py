"""RMSNorm with the residual sum folded in (src/quanta/minimax/model_m3.py:60-65)."""

from __future__ import annotations

import torch

from .. import kernels
from .base import Norm, NormedPending, StreamsPending, TensorSpec, register


@register("norm", "rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    """``weight * x * rsqrt(mean(x^2) + eps)`` with float32 statistics; plain weight (no ``1 + w``)."""

    def __init__(self, width: int, eps: float, weight_name: str, scalar_gain: bool = False):
        """``scalar_gain``: the checkpoint holds ONE number that multiplies every coordinate (a tensor without
        dimensions); it is spread over ``width`` gains at load, so the kernels see the usual vector."""
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.scalar_gain = bool(scalar_gain)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, () if self.scalar_gain else (self.width,), kind="f32", init="gain")]

    def load(self, fetch):
        self.weight = fetch(self.weight_name)
        if self.scalar_gain:
            self.weight = self.weight.reshape(1).expand(self.width).contiguous()

    def forward_streams(self, x, pending, read_w, out, rows=None, store=True):
        if x.dim() == 2:
            x = x.unsqueeze(1)          # one stream
        if pending is not None and not isinstance(pending, StreamsPending):
            raise TypeError(f"several residual streams take a StreamsPending, not {type(pending).__name__}")
        y, mix, out_w, mult = (pending.y, pending.mix, pending.out_w, pending.mult) if pending is not None else (None, None, None, 0.0)
        kernels.streams_mix_rmsnorm(x, y, mix, out_w, mult, read_w, self.weight, self.eps, out, rows=rows, store=store)

    def forward(self, h, delta, out, rows=None, store_h=True):
        if h.dim() == 3 or isinstance(delta, StreamsPending):
            # several residual streams: whoever asks for the plain norm (the output head) reads their sum
            self.forward_streams(h, delta, None, out, rows=rows, store=store_h)
            return
        if isinstance(delta, NormedPending):
            if isinstance(delta.norm, RMSNorm):
                # the norm of the sublayer's output, the sum and this norm in one launch
                normed_add(h, delta, self.weight, self.eps, out, rows, store_h)
                return
            delta = delta.materialize()
        kernels.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows, store_h=store_h)


def normed_add(h, delta: NormedPending, weight, eps: float, out, rows, store_h: bool) -> None:
    """``h += norm(delta)`` and ``out = weight * rms(h)`` (``weight`` None: ``out = h``) in one launch; the addends
    of the sublayer's output (slots, biases, a second branch) are summed there too."""
    a = delta.addends
    kernels.normed_add_rmsnorm(h, a.y, delta.norm.weight, delta.norm.eps, weight, eps, out, rows=rows, store_h=store_h,
                               y_scale=a.scale, y_bias=a.bias, extra=a.extra, extra_scale=a.extra_scale,
                               extra_bias=a.extra_bias)


@register("norm", "none")
class NoNorm(Norm):
    """No norm: the sublayer reads the residual stream as it is.  ``forward`` still takes the pending contribution
    into the stream (in the same launch when it is a normed one) and hands ``out`` the stream in the activation
    dtype."""

    graph_safe = True

    def __init__(self, width: int):
        self.width = int(width)

    def forward(self, h, delta, out, rows=None, store_h=True):
        if h.dim() == 3 or isinstance(delta, StreamsPending):
            raise NotImplementedError("reading several residual streams without a norm is not built")
        if isinstance(delta, NormedPending) and isinstance(delta.norm, RMSNorm):
            normed_add(h, delta, None, 0.0, out, rows, store_h)
            return
        if isinstance(delta, NormedPending):
            delta = delta.materialize()
        if delta is not None:
            kernels.residual_add(h, delta)
        kernels.normed_add_rmsnorm(h, None, None, 0.0, None, 0.0, out, rows=rows, store_h=False)
