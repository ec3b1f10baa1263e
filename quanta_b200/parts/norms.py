"""RMSNorm with the residual sum folded in (src/quanta/minimax/model_m3.py:60-65)."""

from __future__ import annotations

import torch

from .. import kernels
from .base import Norm, NormedPending, StreamCopy, StreamsPending, TensorSpec, register


@register("norm", "rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    """``weight * x * rsqrt(mean(x^2) + eps)`` with float32 statistics; plain weight (no ``1 + w``)."""

    def __init__(self, width: int, eps: float, weight_name: str, scalar_gain: bool = False, groups: int = 1):
        """``scalar_gain``: the checkpoint holds ONE number that multiplies every coordinate (a tensor without
        dimensions); it is spread over ``width`` gains at load, so the kernels see the usual vector.  ``groups``:
        the vector is cut into that many equal consecutive parts and each is divided by its OWN root mean square
        (``eps`` inside each root); the gain still has ``width`` numbers."""
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.scalar_gain = bool(scalar_gain)
        self.groups = int(groups)
        if not 1 <= self.groups <= kernels.NORM_MAX_GROUPS or self.width % self.groups:
            raise ValueError(f"rms_norm: {groups} groups do not divide a width of {width} "
                             f"(1 to {kernels.NORM_MAX_GROUPS})")
        self.weight: torch.Tensor | None = None

    def tensor_specs(self):
        return [TensorSpec(self.weight_name, () if self.scalar_gain else (self.width,), kind="f32", init="gain")]

    def load(self, fetch):
        self.weight = fetch(self.weight_name)
        if self.scalar_gain:
            self.weight = self.weight.reshape(1).expand(self.width).contiguous()

    def forward_streams(self, x, pending, read_w, out, rows=None, store=True):
        if self.groups != 1:
            raise NotImplementedError("a norm in groups over several residual streams is not built")
        if x.dim() == 2:
            x = x.unsqueeze(1)          # one stream
        if pending is not None and not isinstance(pending, StreamsPending):
            raise TypeError(f"several residual streams take a StreamsPending, not {type(pending).__name__}")
        y, mix, out_w, mult = (pending.y, pending.mix, pending.out_w, pending.mult) if pending is not None else (None, None, None, 0.0)
        kernels.streams_mix_rmsnorm(x, y, mix, out_w, mult, read_w, self.weight, self.eps, out, rows=rows, store=store)

    def forward(self, h, delta, out, rows=None, store_h=True):
        if isinstance(delta, StreamCopy):
            delta = None                # nothing is pending; the copy that came with the stream is not needed here
        if h.dim() == 3 or isinstance(delta, StreamsPending):
            # several residual streams: whoever asks for the plain norm (the output head) reads their sum
            self.forward_streams(h, delta, None, out, rows=rows, store=store_h)
            return
        if isinstance(delta, NormedPending):
            if isinstance(delta.norm, RMSNorm):
                # the norm of the sublayer's output, the sum and this norm in one launch
                normed_add(h, delta, self.weight, self.eps, out, rows, store_h, groups=self.groups)
                return
            delta = delta.materialize()
        if self.groups != 1:
            if delta is not None and delta.dtype != torch.float32:
                delta = delta.float()
            kernels.grouped_normed_add(h, y=delta, weight=self.weight, weight_groups=self.groups, eps=self.eps, out=out,
                                       rows=rows, store_h=store_h)
            return
        kernels.add_rmsnorm(h, delta, self.weight, self.eps, out, rows=rows, store_h=store_h)


def normed_add(h, delta: NormedPending, weight, eps: float, out, rows, store_h: bool, groups: int = 1,
               history=None, n_history: int = 0, history_weights=None) -> None:
    """``h += norm(delta)`` and ``out = weight * rms(h)`` (``weight`` None: ``out = h``) in one launch; the addends
    of the sublayer's output (slots, biases, a second branch) are summed there too.  Norms in groups, branches that
    are normed before they are summed, and a stream that becomes a weighted sum of earlier results (``history``)
    take the kernel that knows them."""
    a = delta.addends
    if groups != 1 or delta.norm.groups != 1 or a.branch_normed or history is not None:
        kernels.grouped_normed_add(h, y=a.y, y_scale=a.scale, y_bias=a.bias, y_gain=a.y_gain, extra=a.extra,
                                   extra_scale=a.extra_scale, extra_bias=a.extra_bias, extra_gain=a.extra_gain,
                                   branch_eps=a.branch_eps, gain=delta.norm.weight, groups=delta.norm.groups,
                                   gain_eps=delta.norm.eps, history=history, n_history=n_history,
                                   history_weights=history_weights, weight=weight, weight_groups=groups, eps=eps,
                                   out=out, rows=rows, store_h=store_h)
        return
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
        if isinstance(delta, StreamCopy):
            delta = None
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
