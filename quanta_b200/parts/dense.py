"""Dense feed-forwards: gated, ``down(act(gate x) * (up x))`` with ``act = silu`` (optionally with a bias on each of
the three projections), or in the clamped form ``g = min(gate x, limit)``, ``u = clamp(up x, -limit, limit)``,
``down(g * sigmoid(alpha g) * (u + 1))``; and ungated, ``down(act(up x))`` with ``act`` the square of relu.

The gate and up matrices are held as one, so a step is two library products and one activation kernel.
The result is float32 (the accumulator of the down product), for blocks that norm it before the sum.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Addends, FeedForward, TensorSpec, register


@register("feed_forward", "gated_dense")
class GatedDense(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, inner_size: int, names: dict, activation: str = "silu", biases: bool = False,
                 limit: float = 0.0, alpha: float = 1.0):
        """``names``: gate, up, down, and with ``biases`` gate_b, up_b, down_b (float32 vectors; the down bias is
        handed on as an addend of the output, for the norm kernel that reads it).  ``activation``: ``"silu"`` or
        ``"clamped"`` (with ``limit`` and ``alpha``)."""
        if activation not in ("silu", "clamped"):
            raise ValueError(f"gated_dense: activation {activation!r} is not built (silu and clamped are)")
        if activation == "clamped" and not limit > 0:
            raise ValueError(f"gated_dense: the clamped activation needs a positive limit, got {limit}")
        self.hidden, self.inner, self.names = int(hidden_size), int(inner_size), dict(names)
        self.activation, self.biases, self.limit, self.alpha = activation, bool(biases), float(limit), float(alpha)
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def tensor_specs(self):
        n = self.names
        specs = [TensorSpec(n["gate"], (self.inner, self.hidden)), TensorSpec(n["up"], (self.inner, self.hidden)),
                 TensorSpec(n["down"], (self.hidden, self.inner))]
        if self.biases:
            specs += [TensorSpec(n["gate_b"], (self.inner,), "f32", "bias"), TensorSpec(n["up_b"], (self.inner,), "f32", "bias"),
                      TensorSpec(n["down_b"], (self.hidden,), "f32", "bias")]
        return specs

    def load(self, fetch):
        gate = fetch(self.names["gate"])
        self.w_gate_up = torch.empty((2 * self.inner, self.hidden), dtype=gate.dtype, device=gate.device)
        self.w_gate_up[: self.inner].copy_(gate)
        del gate
        self.w_gate_up[self.inner:].copy_(fetch(self.names["up"]))
        self.w_down = fetch(self.names["down"])
        if self.biases:
            self.b_gate_up = torch.cat([fetch(self.names["gate_b"]), fetch(self.names["up_b"])]).contiguous()
            self.b_down = fetch(self.names["down_b"]).contiguous()

    def forward(self, x, ctx):
        T = x.shape[0]
        gate_up = linear(x, self.w_gate_up)
        act = empty_rows(T, self.inner, dtype=x.dtype, device=x.device)
        if self.activation == "silu" and not self.biases:
            kernels.silu_mul(gate_up, act)
        else:
            kernels.glu_act(gate_up, act, bias=self.b_gate_up, limit=self.limit, alpha=self.alpha,
                            kind=kernels.GLU_CLAMPED if self.activation == "clamped" else kernels.GLU_SILU)
        y = linear(act, self.w_down, out_dtype=torch.float32)
        return Addends(y, bias=self.b_down) if self.biases else y


@register("feed_forward", "ungated_dense")
class UngatedDense(FeedForward):
    """``down(act(up x))``; ``activation``: ``"relu_squared"`` (``relu(z)^2``)."""

    graph_safe = True

    def __init__(self, hidden_size: int, inner_size: int, names: dict, activation: str = "relu_squared"):
        if activation != "relu_squared":
            raise ValueError(f"ungated_dense: activation {activation!r} is not built (relu_squared is)")
        self.hidden, self.inner, self.names = int(hidden_size), int(inner_size), dict(names)   # up, down
        self.w_up = self.w_down = None

    def tensor_specs(self):
        n = self.names
        return [TensorSpec(n["up"], (self.inner, self.hidden)), TensorSpec(n["down"], (self.hidden, self.inner))]

    def load(self, fetch):
        self.w_up, self.w_down = fetch(self.names["up"]), fetch(self.names["down"])

    def forward(self, x, ctx):
        T = x.shape[0]
        up = linear(x, self.w_up)
        act = empty_rows(T, self.inner, dtype=x.dtype, device=x.device)
        kernels.relu_squared(up, act)
        return linear(act, self.w_down, out_dtype=torch.float32)
