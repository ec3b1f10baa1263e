"""Selective state-space mixer, and two mixers side by side.

``selective_scan``: ``[u | z] = W_in x`` (``inner`` channels each); ``u`` passes a short causal convolution per
channel with a bias and silu; ``[low | B | C] = W_x u`` (``dt_rank``, ``state``, ``state`` numbers a token);
``dt = softplus(W_dt low + b)`` per channel; with ``A = -exp(A_log)`` ``[inner, state]`` and ``D`` per channel

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n          y_c = sum_n S[c, n] C_n + D_c u_c

then ``y * silu(z)`` and ``W_o``.  ``S`` (float32, zero at admission) and the convolution's last ``taps - 1``
inputs are per-request state.  Step sizes, decays, the state and the gate are float32; the projections are
library products whose float32 accumulators feed the kernels (the step projection multiplies the float32 ``low``
with the float32 copy of ``W_dt``; its bias and softplus are applied inside the scan).

``parallel_mixers``: two mixers read the same input; the result is ``left_scale * left + right_scale * right``,
or with ``left_norm`` / ``right_norm`` ``left_scale * norm_l(left) + right_scale * norm_r(right)`` (each branch
RMS-normed over the whole width with a gain of its own first).  Their caches and states live side by side (stream
and state names must differ); the sum, and the branch norms, are left to the norm kernel that reads the mixer's
output when the block has one.  The two branches share nothing but their input, so the right one runs on a second
CUDA stream beside the left one (``concurrent``; the streams fork and join inside the launch order, also in a captured
step): an attention that fills the SMs and a recurrence that is a chain in time with few warps overlap.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import Addends, Mixer, TensorSpec, make, register, run_beside


@register("mixer", "selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, inner: int, n_state: int, dt_rank: int, conv_taps: int, names: dict,
                 state_name: str = "scan_state", conv_state_name: str = "scan_conv_inputs"):
        if inner <= 0 or dt_rank <= 0 or conv_taps < 1:
            raise ValueError("selective_scan: inner, dt_rank and conv_taps must be positive")
        if not 0 < n_state <= kernels.SCAN_MAX_STATE:
            raise ValueError(f"selective_scan: a state of {n_state} per channel is outside the kernel's 1 to "
                             f"{kernels.SCAN_MAX_STATE}")
        self.hidden, self.inner, self.N, self.R, self.taps = int(hidden_size), int(inner), int(n_state), int(dt_rank), int(conv_taps)
        self.names, self.state_name, self.conv_state_name = dict(names), state_name, conv_state_name
        # in, conv, conv_b, x, dt, dt_b, A_log, D, o
        self.w_in = self.conv_w = self.conv_b = self.w_x = self.w_dt = self.dt_b = self.A = self.D = self.w_o = None

    def tensor_specs(self):
        n, W, C = self.names, self.hidden, self.inner
        return [TensorSpec(n["in"], (2 * C, W)), TensorSpec(n["conv"], (C, self.taps), "f32", "normal"),
                TensorSpec(n["conv_b"], (C,), "f32", "bias"), TensorSpec(n["x"], (self.R + 2 * self.N, C)),
                TensorSpec(n["dt"], (C, self.R), "f32", "normal"), TensorSpec(n["dt_b"], (C,), "f32", "bias"),
                TensorSpec(n["A_log"], (C, self.N), "f32", "gain"), TensorSpec(n["D"], (C,), "f32", "gain"),
                TensorSpec(n["o"], (W, C))]

    def load(self, fetch):
        n = self.names
        self.w_in = fetch(n["in"])
        self.conv_w, self.conv_b = fetch(n["conv"]).contiguous(), fetch(n["conv_b"]).contiguous()
        w_x = fetch(n["x"])
        rows = -(-w_x.shape[0] // 8) * 8               # product rows that start on 16 bytes
        self.w_x = torch.zeros((rows, self.inner), dtype=w_x.dtype, device=w_x.device)
        self.w_x[: w_x.shape[0]].copy_(w_x)
        self.w_dt, self.dt_b = fetch(n["dt"]).contiguous(), fetch(n["dt_b"]).contiguous()
        self.A = (-torch.exp(fetch(n["A_log"]).float())).contiguous()
        self.D, self.w_o = fetch(n["D"]).contiguous(), fetch(n["o"])

    def state_spec(self):
        return {self.state_name: ((self.inner, self.N), torch.float32),
                self.conv_state_name: ((self.taps - 1, self.inner), torch.float32)}

    def forward(self, x, ctx, cache, state):
        T, C = x.shape[0], self.inner
        uz = linear(x, self.w_in, out_dtype=torch.float32)
        u = empty_rows(T, C, dtype=x.dtype, device=x.device)
        kernels.short_conv(uz[:, :C], self.conv_w, state[self.conv_state_name], u, ctx.tok_req, ctx.req_start,
                           ctx.req_slot, bias=self.conv_b, silu=True)
        proj = linear(u, self.w_x, out_dtype=torch.float32)
        y = empty_rows(T, C, dtype=x.dtype, device=x.device)
        dt_pre = linear(proj[:, : self.R], self.w_dt)          # float32 operands: a true float32 product
        kernels.selective_scan(u, proj, uz[:, C:], dt_pre, self.dt_b, self.A, self.D, state[self.state_name], y,
                               ctx.req_start, ctx.req_slot, self.R, self.N)
        return linear(y, self.w_o, out_dtype=torch.float32)


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    graph_safe = True

    def __init__(self, left, right, left_scale: float = 1.0, right_scale: float = 1.0, left_norm=None,
                 right_norm=None, concurrent: bool = True):
        self.concurrent = bool(concurrent)
        self.left, self.right = make("mixer", left), make("mixer", right)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self.left_norm = make("norm", left_norm) if left_norm is not None else None
        self.right_norm = make("norm", right_norm) if right_norm is not None else None
        for n in (self.left_norm, self.right_norm):
            if n is not None and (not hasattr(n, "weight") or getattr(n, "groups", 1) != 1):
                raise ValueError("parallel_mixers: a branch norm is an rms_norm over the whole width")
        if self.left_norm is not None and self.right_norm is not None and self.left_norm.eps != self.right_norm.eps:
            raise ValueError("parallel_mixers: the two branch norms share one eps")
        self.graph_safe = bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def children(self):
        return [p for p in (self.left, self.right, self.left_norm, self.right_norm) if p is not None]

    def cache_spec(self):
        specs = []
        for m in (self.left, self.right):
            need = m.cache_spec()
            if need is not None:
                specs += list(need) if isinstance(need, (tuple, list)) else [need]
        return None if not specs else specs[0] if len(specs) == 1 else tuple(specs)

    def state_spec(self):
        spec = dict(self.left.state_spec())
        for name, need in self.right.state_spec().items():
            if name in spec:
                raise ValueError(f"both mixers keep a state named {name!r}")
            spec[name] = need
        return spec

    def forward(self, x, ctx, cache, state):
        if self.concurrent and x.is_cuda:
            b, a = run_beside(lambda: self.right.forward(x, ctx, cache, state),
                              lambda: self.left.forward(x, ctx, cache, state), x.device)
        else:
            a = self.left.forward(x, ctx, cache, state)
            b = self.right.forward(x, ctx, cache, state)
        a = a if isinstance(a, Addends) else Addends(a)
        b = b if isinstance(b, Addends) else Addends(b)
        if a.extra is not None or a.y.dim() != 2 or a.branch_normed or (self.left_norm is not None and a.scale != 1.0):
            a = Addends(a.total())
        if b.extra is not None or b.y.dim() != 2 or b.scale != 1.0 or b.branch_normed:
            b = Addends(b.total())
        eps = (self.left_norm or self.right_norm).eps if (self.left_norm or self.right_norm) is not None else 0.0
        return Addends(a.y, scale=a.scale * self.left_scale, bias=a.bias, extra=b.y, extra_scale=self.right_scale,
                       extra_bias=b.bias, y_gain=None if self.left_norm is None else self.left_norm.weight,
                       extra_gain=None if self.right_norm is None else self.right_norm.weight, branch_eps=eps)
