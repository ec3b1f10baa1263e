"""Grouped-query softmax attention over the paged cache.

Formula, in order (src/quanta/minimax/attention.py:166-204): q/k/v projections without bias; q/k
RMSNorm before the rotation, either over the concatenated heads (``"per_layer"``, weight
``[heads*head_dim]``) or per head (``"per_head"``, weight ``[head_dim]``); rotation of the first
``rotary_dim`` dims by the position encoding part; K (rotated) and V appended to the cache; scores
``q.k * scale`` over the keys at positions <= the query's (and inside the window, if any), softmax in
float32, ``P V``; output projection.  q head ``h`` reads kv head ``h // (n_q / n_kv)``.

Options beside that formula, all off by default: values of another head size than the keys
(``value_dim``); a query temperature ``q *= 1 + coef * ln(floor((p + 1) / every) + 1)`` at position p
(``q_temperature``); a gate per head, ``out_h *= sigmoid(W_g x)_h`` before the output projection (tensor
``names["g"]``, ``[heads, hidden]``, part of the fused input projection); a layer without keys and values
of its own (``own_kv`` False: no k/v tensors; the model's run order names the entry whose cache it reads); a short
causal convolution over time on every channel of the projected q, k and v, before norm and rotation (``conv_taps``
> 0; tensors ``names["q_conv"]`` / ``k_conv`` / ``v_conv`` ``[channels, taps]``, no bias; the last ``taps - 1``
projected rows of a request are per-request state, so a portion that starts anywhere sees what the whole prompt
sees); a learned number per q head that multiplies the head's scores (tensor ``names["head_temperature"]``
``[heads]``, float32; folded into the normed, rotated query); softmax weights that stay 32-bit on the tensor
cores too (``float32_weights``: the kernels that feed ``P V`` with the weights in two bfloat16 parts, and float32
arithmetic for single tokens, instead of the kernels that round the weights to bfloat16).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..matmul import empty_rows, linear
from .base import CacheSpec, CacheStream, KeepAll, Mixer, TensorSpec, Window, make, register

_NORM_KIND = {None: kernels.NORM_NONE, "per_layer": kernels.NORM_PER_LAYER, "per_head": kernels.NORM_PER_HEAD}


@register("mixer", "gqa_attention")
class GQAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 position, qk_norm: str | None, qk_norm_eps: float, names: dict, window: int | None = None,
                 value_dim: int | None = None, q_temperature: tuple | None = None, own_kv: bool = True,
                 float32_output: bool = False, conv_taps: int = 0, conv_state_name: str = "attention_conv_inputs",
                 float32_weights: bool = False):
        if n_q_heads % n_kv_heads:
            raise ValueError(f"{n_q_heads} q heads are not a multiple of {n_kv_heads} kv heads")
        value_dim = head_dim if value_dim is None else int(value_dim)
        if not 0 < head_dim <= 256 or not 0 < value_dim <= 256:
            raise ValueError(f"head sizes {head_dim} / {value_dim}: the attention kernels take 1 to 256")
        if qk_norm not in _NORM_KIND:
            raise ValueError(f"qk_norm {qk_norm!r} is not None, 'per_layer' or 'per_head'")
        self.hidden, self.nq, self.nkv, self.hd = int(hidden_size), int(n_q_heads), int(n_kv_heads), int(head_dim)
        self.vd, self.own_kv, self.float32_output = value_dim, bool(own_kv), bool(float32_output)
        self.scale, self.qk_norm, self.eps = float(scale), qk_norm, float(qk_norm_eps)
        self.window = window
        self.q_temp = (0.0, 0) if q_temperature is None else (float(q_temperature[0]), int(q_temperature[1]))
        if self.q_temp[1] < 0:
            raise ValueError(f"q_temperature every {self.q_temp[1]} must be positive (0: none)")
        self.position = make("position", position) if isinstance(position, tuple) else position
        self.names = dict(names)      # q, o; k, v with own_kv; q_norm (k_norm) when normed; g for a gate per head
        self.gated = "g" in self.names
        self.taps, self.conv_state_name = int(conv_taps), conv_state_name
        if self.taps < 0 or (self.taps and (not self.own_kv or self.gated)):
            raise ValueError("gqa_attention: the convolution on q, k, v needs keys and values of the layer's own and "
                             "no gate per head")
        self.conv_w = self.head_temp = None
        self.float32_weights = bool(float32_weights)
        # the tensor-core kernels take equal key and value head sizes that are multiples of 16
        self.mma_shapes = self.hd == self.vd and self.hd % 16 == 0
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        # more q heads per kv head than the single-token kernel takes: single tokens run as portions of one,
        # whose tile list comes from the host each step, so such a model's decode steps are not captured
        self.graph_safe = self.float32_weights or self.nq // self.nkv <= kernels.ATTN_DECODE_MAX_GROUP

    def children(self):
        return [self.position]

    def tensor_specs(self):
        n, H, hd, vd = self.names, self.hidden, self.hd, self.vd
        specs = [TensorSpec(n["q"], (self.nq * hd, H)), TensorSpec(n["o"], (H, self.nq * vd))]
        if self.own_kv:
            specs += [TensorSpec(n["k"], (self.nkv * hd, H)), TensorSpec(n["v"], (self.nkv * vd, H))]
        if self.gated:
            specs.append(TensorSpec(n["g"], (self.nq, H)))
        if self.qk_norm is not None:
            specs.append(TensorSpec(n["q_norm"], (self.nq * hd if self.qk_norm == "per_layer" else hd,), "f32", "gain"))
            if self.own_kv:
                specs.append(TensorSpec(n["k_norm"], (self.nkv * hd if self.qk_norm == "per_layer" else hd,), "f32", "gain"))
        if self.taps:
            specs += [TensorSpec(n["q_conv"], (self.nq * hd, self.taps), "f32", "conv"),
                      TensorSpec(n["k_conv"], (self.nkv * hd, self.taps), "f32", "conv"),
                      TensorSpec(n["v_conv"], (self.nkv * vd, self.taps), "f32", "conv")]
        if "head_temperature" in n:
            specs.append(TensorSpec(n["head_temperature"], (self.nq,), "f32", "gain"))
        return specs

    def load(self, fetch):
        n = self.names
        q = fetch(n["q"])
        # the rows of the fused input projection: q, then k and v where the layer has its own, then the gates;
        # padded to a multiple of 8 so that every row of the product starts on 16 bytes
        a = self.nq * self.hd
        b = a + (self.nkv * self.hd if self.own_kv else 0)
        c = b + (self.nkv * self.vd if self.own_kv else 0)
        self.gate_off = c
        rows = c + (self.nq if self.gated else 0)
        self.w_qkv = torch.zeros((-(-rows // 8) * 8, self.hidden), dtype=q.dtype, device=q.device)
        self.w_qkv[:a].copy_(q)
        del q
        if self.own_kv:
            self.w_qkv[a:b].copy_(fetch(n["k"]))
            self.w_qkv[b:c].copy_(fetch(n["v"]))
        if self.gated:
            self.w_qkv[c:rows].copy_(fetch(n["g"]))
        self.w_o = fetch(n["o"])
        if self.qk_norm is not None:
            self.q_norm_w = fetch(n["q_norm"])
            self.k_norm_w = fetch(n["k_norm"]) if self.own_kv else None
        if self.taps:
            self.conv_w = torch.cat([fetch(n["q_conv"]), fetch(n["k_conv"]), fetch(n["v_conv"])], 0).contiguous()
        if "head_temperature" in n:
            self.head_temp = fetch(n["head_temperature"]).contiguous()

    @property
    def conv_channels(self) -> int:
        return self.nq * self.hd + self.nkv * (self.hd + self.vd)

    def state_spec(self):
        if self.taps > 1:
            return {self.conv_state_name: ((self.taps - 1, self.conv_channels), torch.float32)}
        return {}

    def cache_spec(self):
        if not self.own_kv:
            return None
        return CacheSpec((CacheStream("k", self.nkv, self.hd), CacheStream("v", self.nkv, self.vd)),
                         KeepAll() if self.window is None else Window(int(self.window)))

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        if self.taps:
            # the projection's float32 accumulators pass the convolution and reach norm and rotation unrounded
            proj = linear(x, self.w_qkv, out_dtype=torch.float32)
            C = self.conv_channels
            qkv = torch.empty((T, C), dtype=torch.float32, device=x.device)
            hist = state[self.conv_state_name] if self.taps > 1 else \
                torch.empty((0, 0, C), dtype=torch.float32, device=x.device)
            kernels.short_conv(proj[:, :C], self.conv_w, hist, qkv, ctx.tok_req, ctx.req_start, ctx.req_slot, plain=True)
        else:
            qkv = linear(x, self.w_qkv)
        q = torch.empty((T, self.nq, self.hd), dtype=x.dtype, device=x.device)
        tables = self.position.rotary_tables(x.device)
        if tables is None:
            inv_freq = torch.empty(0, dtype=torch.float32, device=x.device)
            pair_axis, rd = None, 0
        else:
            inv_freq, pair_axis, rd, n_axes = tables
            if ctx.positions.dim() != 2 or ctx.positions.shape[1] < n_axes:
                raise ValueError(f"the position encoding reads {n_axes} position axes; the step gives "
                                 f"{tuple(ctx.positions.shape)}")
        if cache is None or (cache.write and not self.own_kv):
            raise ValueError("an attention layer without keys and values of its own must be given another "
                             "entry's cache to read (ScheduleEntry.read_cache_of)")
        if tuple(cache.k.shape[1:]) != (self.nkv, cache.page_size, self.hd) or cache.v.shape[3] != self.vd:
            raise ValueError(f"the cache holds keys {tuple(cache.k.shape[1:])} and values of {cache.v.shape[3]}; this "
                             f"layer reads {self.nkv} heads of {self.hd} / {self.vd}")
        kernels.qknorm_rope_write(
            qkv, q, cache.k if cache.write else None, cache.v if cache.write else None, self.q_norm_w,
            self.k_norm_w, _NORM_KIND[self.qk_norm], self.eps, inv_freq, pair_axis, ctx.positions, ctx.tok_pos,
            ctx.tok_req, cache.block_table, self.nq, self.nkv, self.hd, rd, cache.page_size, ctx.status,
            vd=self.vd, has_kv=self.own_kv, q_temp_coef=self.q_temp[0], q_temp_every=self.q_temp[1],
            head_scale=self.head_temp)
        out = empty_rows(T, self.nq, self.vd, dtype=x.dtype, device=x.device)
        self.attend(q, cache, out, ctx)
        if self.gated:
            kernels.head_sigmoid_gate(out, qkv[:, self.gate_off: self.gate_off + self.nq], self.nq, self.vd)
        return linear(out.view(T, self.nq * self.vd), self.w_o,
                      out_dtype=torch.float32 if self.float32_output else None)

    def attend(self, q, cache, out, ctx):
        """float32 (and head sizes the tensor-core kernels do not take: keys and values of different sizes, or
        no multiple of 16): the SIMT kernel, every token alike.  bfloat16: tensor-core kernels, one for single
        tokens (the keys of all of them dealt evenly over the SMs) and one for portions (tiles of
        token-by-head rows)."""
        window = self.window or 0
        if self.float32_weights:
            # scores and weights in float32 whatever the dtype: portions of shapes the tensor cores take run there
            # with the weights in two bfloat16 parts; single tokens cut their keys into ranges that are joined
            R = int(ctx.req_start.numel()) - 1
            warps = max(1, q.shape[0] * self.nkv)
            # about 2,048 warps in all, at least 32 keys a range (measured on a B200 with 4 kv heads of 128: 8 tokens
            # over 2,048 keys 47 us with 64 ranges against 63 with 32; 32 tokens 120 us with 16 against 150 with 64; one
            # token over 8,192 keys 61 us with 256 against 110 with 64)
            n_split = max(1, min(-(-2048 // warps), -(-max(1, ctx.max_len_after) // 32), 256))
            kernels.window_attention(q, cache.k, cache.v, out, ctx.tok_pos, ctx.tok_req, cache.block_table, self.scale,
                                     window, ctx.status, n_split=n_split, n_requests=R)
            return
        if q.dtype != torch.bfloat16 or not self.mma_shapes:
            kernels.paged_attention_simt(q, cache.k, cache.v, out, ctx.tok_pos, ctx.tok_req, cache.block_table,
                                         self.scale, window, ctx.status)
            return
        dec_tok, n_dec, spans = step_work(ctx, q.device)
        G = self.nq // self.nkv
        if n_dec and G > kernels.ATTN_DECODE_MAX_GROUP:
            # more q heads per kv head than the single-token kernel takes: such a token is a portion of one
            starts = ctx.host.get("req_start") or [0, ctx.n_tokens]
            spans = [(r, starts[r], starts[r + 1] - starts[r]) for r in range(len(starts) - 1)]
            n_dec = 0
        if n_dec:
            n_parts = kernels.attn_decode_parts(self.nkv, max(1, ctx.max_len_after))
            part_o = torch.empty(n_dec * self.nq * n_parts * self.hd, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(n_dec * self.nq * n_parts * 2, dtype=torch.float32, device=q.device)
            kernels.attn_decode(q, cache.k, cache.v, out, part_o, part_ml, dec_tok, n_dec, ctx.tok_pos, ctx.tok_req,
                                cache.block_table, self.scale, window, n_parts, ctx.status)
        if spans:
            key = ("span_tiles", G, self.hd, kernels.attn_span_rows(self.hd, self.nq, self.nkv, cache.page_size))
            if key not in ctx.work:
                rows = kernels.attn_span_rows(self.hd, self.nq, self.nkv, cache.page_size)
                tiles = [[r, t0, n, r0] for (r, t0, n) in spans for r0 in range(0, n * G, rows)]
                # tiles that read the most keys first: the short ones fill the SMs at the end
                after = ctx.host.get("req_len_after")
                if after is not None:
                    tiles.sort(key=lambda t: -(after[t[0]] - t[2] + min(t[2], (t[3] + rows) // G)))
                ctx.work[key] = torch.tensor(tiles, dtype=torch.int32).to(q.device, non_blocking=True)
            kernels.attn_span(q, cache.k, cache.v, out, ctx.tok_pos, cache.block_table, ctx.work[key], self.scale,
                              window, ctx.status)


def step_work(ctx, device):
    """(token rows of single-token requests, their number, portions of the other requests)."""
    if ctx.spans is None and ctx.dec_tok is None:
        starts = ctx.host.get("req_start") or [0, ctx.n_tokens]
        dec, spans = [], []
        for r in range(len(starts) - 1):
            n = starts[r + 1] - starts[r]
            (dec.append(starts[r]) if n == 1 else spans.append((r, starts[r], n)))
        ctx.spans, ctx.n_dec = spans, len(dec)
        ctx.dec_tok = torch.tensor(dec, dtype=torch.int32).to(device, non_blocking=True) if dec else None
    return ctx.dec_tok, ctx.n_dec, ctx.spans or []
