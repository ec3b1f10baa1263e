"""Gated delta rule: a linear recurrence per head whose state is a matrix S [key channel, value channel], with one
decay and one write strength per (token, head).

With q, k = W_q x, W_k x (``n_groups`` x ``dim`` each; head h reads group ``h // (n_heads / n_groups)``) and
v = W_v x (``n_heads`` x ``value_dim``), each passed through a short causal convolution over time per channel (no
bias) and silu; q and k made unit vectors per group, ``z / sqrt(sum(z^2) + unit_eps)``, q also times ``q_scale``;
``beta = sigmoid(W_b x)`` and ``g = exp(-exp(A_log) * softplus(W_a x + dt_bias))`` per head:

    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

Each head's o is divided by its root mean square over ``value_dim``, multiplied by a gain that the heads share and
by ``silu(W_g x)``, and projected by W_o.  S (float32, zero at admission) and the convolution's last ``taps - 1``
inputs are per-request state.  All projections that read x are one library product whose float32 accumulators feed
the kernels; everything from there to the gated result is float32.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Mixer, TensorSpec, register


@register("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_heads: int, n_groups: int, dim: int, value_dim: int, conv_taps: int,
                 q_scale: float, unit_eps: float, norm_eps: float, names: dict, state_name: str = "gated_delta_state",
                 conv_state_name: str = "gated_delta_conv_inputs"):
        if n_heads <= 0 or n_groups <= 0 or n_heads % n_groups:
            raise ValueError(f"gated_delta_rule: {n_heads} heads are not a positive multiple of {n_groups} groups")
        if not 0 < dim <= kernels.GATED_DELTA_MAX_DIM or not 0 < value_dim <= kernels.GATED_DELTA_MAX_DIM:
            raise ValueError(f"gated_delta_rule: head sizes {dim} / {value_dim} outside the kernel's 1 to "
                             f"{kernels.GATED_DELTA_MAX_DIM}")
        if conv_taps < 0:
            raise ValueError("gated_delta_rule: a convolution of a negative number of taps")
        self.hidden, self.H, self.G, self.D, self.DV = int(hidden_size), int(n_heads), int(n_groups), int(dim), int(value_dim)
        self.taps, self.q_scale, self.unit_eps, self.norm_eps = int(conv_taps), float(q_scale), float(unit_eps), float(norm_eps)
        # q, k, v, g (the output gate), b, a, A_log, dt_bias, norm, o; q_conv, k_conv, v_conv with a convolution
        self.names, self.state_name, self.conv_state_name = dict(names), state_name, conv_state_name
        self.n_conv = 2 * self.G * self.D + self.H * self.DV            # channels of [q | k | v]
        self.gate_off = self.n_conv
        self.b_off = self.gate_off + self.H * self.DV
        self.a_off = self.b_off + self.H
        self.w_in = self.conv_w = self.A_log = self.dt_bias = self.gain = self.w_o = None

    def tensor_specs(self):
        n, W, GD, HV = self.names, self.hidden, self.G * self.D, self.H * self.DV
        specs = [TensorSpec(n["q"], (GD, W)), TensorSpec(n["k"], (GD, W)), TensorSpec(n["v"], (HV, W)),
                 TensorSpec(n["g"], (HV, W)), TensorSpec(n["b"], (self.H, W)), TensorSpec(n["a"], (self.H, W)),
                 TensorSpec(n["A_log"], (self.H,), "f32", "gain"), TensorSpec(n["dt_bias"], (self.H,), "f32", "bias"),
                 TensorSpec(n["norm"], (self.DV,), "f32", "gain"), TensorSpec(n["o"], (W, HV))]
        if self.taps:
            specs += [TensorSpec(n["q_conv"], (GD, self.taps), "f32", "conv"),
                      TensorSpec(n["k_conv"], (GD, self.taps), "f32", "conv"),
                      TensorSpec(n["v_conv"], (HV, self.taps), "f32", "conv")]
        return specs

    def load(self, fetch):
        n = self.names
        first = fetch(n["q"])
        rows = self.a_off + self.H
        # the rows of the fused input projection, padded so that every row of the product starts on 16 bytes
        self.w_in = torch.zeros((-(-rows // 8) * 8, self.hidden), dtype=first.dtype, device=first.device)
        at = 0
        for key in ("q", "k", "v", "g", "b", "a"):
            w = first if key == "q" else fetch(n[key])
            self.w_in[at: at + w.shape[0]].copy_(w)
            at += w.shape[0]
        del first
        self.A_log, self.dt_bias = fetch(n["A_log"]).contiguous(), fetch(n["dt_bias"]).contiguous()
        self.gain, self.w_o = fetch(n["norm"]).contiguous(), fetch(n["o"])
        if self.taps:
            self.conv_w = torch.cat([fetch(n["q_conv"]), fetch(n["k_conv"]), fetch(n["v_conv"])], 0).contiguous()
        else:
            # no convolution: one tap of weight one, so that the same kernel applies the activation
            self.conv_w = torch.ones((self.n_conv, 1), dtype=torch.float32, device=self.gain.device)

    def state_spec(self):
        spec = {self.state_name: ((self.H, self.D, self.DV), torch.float32)}
        if self.taps > 1:
            spec[self.conv_state_name] = ((self.taps - 1, self.n_conv), torch.float32)
        return spec

    def forward(self, x, ctx, cache, state):
        T, C = x.shape[0], self.n_conv
        proj = linear(x, self.w_in, out_dtype=torch.float32)
        qkv = torch.empty((T, C), dtype=torch.float32, device=x.device)
        hist = state[self.conv_state_name] if self.taps > 1 else \
            torch.empty((0, 0, C), dtype=torch.float32, device=x.device)
        kernels.short_conv(proj[:, :C], self.conv_w, hist, qkv, ctx.tok_req, ctx.req_start, ctx.req_slot, silu=True)
        o = torch.empty((T, self.H, self.DV), dtype=torch.float32, device=x.device)
        kernels.gated_delta(qkv, proj, self.a_off, self.b_off, self.A_log, self.dt_bias, state[self.state_name], o,
                            ctx.req_start, ctx.req_slot, self.H, self.G, self.D, self.DV, self.q_scale, self.unit_eps)
        y = empty_rows(T, self.H * self.DV, dtype=x.dtype, device=x.device)
        kernels.head_norm_gate(o, proj, self.gate_off, self.gain, y, self.H, self.DV, self.norm_eps, gate="silu")
        return linear(y, self.w_o, out_dtype=torch.float32)
