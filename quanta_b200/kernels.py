"""Python face of the CUDA kernels: argument checks, pointers, launch on torch's current stream.

Every function here launches hand-written sm_100a code from ``csrc``; there is no CPU or library
fallback, and a missing or unbuildable extension raises at the first call.  Tensors must be CUDA,
contiguous and of the stated dtype; a violated precondition is a ``ValueError`` before anything is
launched.
"""

from __future__ import annotations

import ctypes
import os

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
NORM_NONE, NORM_PER_LAYER, NORM_PER_HEAD = 0, 1, 2

_STATUS_TEXT = {1: "token id outside the vocabulary", 2: "page id outside the pool (block table)",
                3: "expert id outside the expert table", 4: "a bounded device wait ran out",
                5: "the decode attention scratch has too few entries per row",
                6: "a request's state slot on the device is free or at another position than the host's record",
                7: "a position beyond the table of learned position vectors"}
_KERNEL_TEXT = {1: "embedding", 2: "rope/cache write", 3: "paged attention", 4: "expert plan",
                5: "expert product", 6: "decode attention", 7: "prefill attention", 8: "state slots"}


class KernelError(RuntimeError):
    pass


def lib(unit: str | None = None):
    """The kernel library (entry points as attributes; a unit of kernels is compiled and loaded at the first
    call into it).  ``unit``: build and load that unit now."""
    return _build.load(unit)


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"dtype {t.dtype} is not float32 or bfloat16") from None


def _p(t: torch.Tensor | None):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise ValueError("kernel arguments must be CUDA tensors")
    if not t.is_contiguous():
        raise ValueError("kernel arguments must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """torch's current stream of the current device, as a cudaStream_t."""
    if _raw_stream is not None:       # the same answer as below, without building a Stream object each launch
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0        # kernels of this library launched so far (a plain counter; reset it to count a region)


def _check(rc: int, what: str, n_kernels: int = 1) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += n_kernels
        return
    if rc == -1:
        raise ValueError(f"{what}: bad argument")
    if rc == -2:
        raise ValueError(f"{what}: a size outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {rc}")


def _want(t: torch.Tensor, dtype, name: str) -> None:
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def new_status(device) -> torch.Tensor:
    """Status words the kernels write when they meet an index they cannot honour."""
    return torch.zeros(4, dtype=torch.int32, device=device)


def raise_on_status(status_host) -> None:
    code = int(status_host[0])
    if code:
        raise KernelError(f"device reported: {_STATUS_TEXT.get(code, code)} (value {int(status_host[1])}) in "
                          f"{_KERNEL_TEXT.get(int(status_host[2]), 'kernel ' + str(int(status_host[2])))}")


# ------------------------------------------------------------------------------------------------
def embedding(h: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, status: torch.Tensor,
              scale: float = 1.0, pos_table: torch.Tensor | None = None, tok_pos: torch.Tensor | None = None) -> None:
    """``h[t] = float32(table[ids[t]]) * scale (+ float32(pos_table[tok_pos[t]]))``; ``h`` ``[T, H]``, or
    ``[T, S, H]`` for a model with S residual streams, which all start as the same row."""
    _want(h, torch.float32, "h"); _want(ids, torch.int32, "ids")
    T, H = h.shape[0], h.shape[-1]
    copies = h.shape[1] if h.dim() == 3 else 1
    V = table.shape[0]
    if table.shape[1] != H or ids.numel() != T:
        raise ValueError("embedding: shape mismatch")
    n_pos = 0
    if pos_table is not None:
        _want(tok_pos, torch.int32, "tok_pos")
        if pos_table.shape[1] != H or pos_table.dtype != table.dtype or tok_pos.numel() != T:
            raise ValueError("embedding: the position table does not fit")
        n_pos = pos_table.shape[0]
    _check(lib().qb_embedding(_p(h), _p(table), _code(table), _p(ids), T, H, V, ctypes.c_float(scale), _p(pos_table),
                              _p(tok_pos) if pos_table is not None else ctypes.c_void_p(0), n_pos, copies, _p(status),
                              _stream()), "embedding")


MAX_STREAMS = 16


def streams_mix_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, mix: torch.Tensor | None,
                        out_w: torch.Tensor | None, mult: float, read_w: torch.Tensor | None,
                        weight: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                        rows: torch.Tensor | None = None, store: bool = True) -> None:
    """What lies between two sublayers of a model with several residual streams ``x`` ``[T, S, H]`` (float32), in
    one launch: with ``delta`` (``[T, H]`` or ``[T, K, H]``, K partial results added in order) the write-back
    ``x'_t = sum_s mix[s, t] x_s + mult * out_w[t] * delta`` (stored when ``store``); then the read
    ``u = sum_t read_w[t] x'_t`` (``read_w`` None: the plain sum of the streams) and
    ``out = weight * u * rsqrt(mean(u^2) + eps)`` (``weight`` None: ``u`` itself; ``out`` None: only the
    write-back).  ``rows`` (int32) selects token rows; ``out`` then has one row per entry."""
    _want(x, torch.float32, "x")
    if x.dim() != 3 or x.shape[1] > MAX_STREAMS:
        raise ValueError(f"streams_mix_rmsnorm: x must be [T, S, H] with S <= {MAX_STREAMS}")
    T, S, H = x.shape
    K = 1
    if delta is not None:
        K = delta.shape[1] if delta.dim() == 3 else 1
        if delta.shape[0] != T or delta.shape[-1] != H:
            raise ValueError("streams_mix_rmsnorm: delta shape mismatch")
        _want(mix, torch.float32, "mix"); _want(out_w, torch.float32, "out_w")
        if tuple(mix.shape) != (S, S) or out_w.numel() != S:
            raise ValueError("streams_mix_rmsnorm: mix must be [S, S] and out_w [S]")
    for t, n, size in ((read_w, "read_w", S), (weight, "weight", H)):
        if t is not None:
            _want(t, torch.float32, n)
            if t.numel() != size:
                raise ValueError(f"streams_mix_rmsnorm: {n} has {t.numel()} elements, expected {size}")
    n = T if rows is None else rows.numel()
    if rows is not None:
        _want(rows, torch.int32, "rows")
    if out is not None and (out.shape[0] != n or out.shape[1] != H):
        raise ValueError("streams_mix_rmsnorm: out shape mismatch")
    _check(lib().qb_streams_mix_rmsnorm(_p(x), S, _p(delta), _code(delta) if delta is not None else F32, K,
                                        _p(mix) if delta is not None else ctypes.c_void_p(0),
                                        _p(out_w) if delta is not None else ctypes.c_void_p(0), ctypes.c_float(mult),
                                        _p(read_w), _p(weight), _p(out), _code(out) if out is not None else F32,
                                        _p(rows), n, H, ctypes.c_float(eps), int(store), _stream()),
           "streams_mix_rmsnorm")


def relu_squared(x: torch.Tensor, out: torch.Tensor) -> None:
    """``out = relu(x)^2`` elementwise (float32 inside, one rounding)."""
    if out.shape != x.shape or out.dtype != x.dtype:
        raise ValueError("relu_squared: shape/dtype mismatch")
    _check(lib().qb_relu_squared(_p(x), _p(out), _code(x), ctypes.c_longlong(x.numel()), _stream()), "relu_squared")


def head_sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, n_heads: int, dim: int) -> None:
    """``x[t, h, :] *= sigmoid(gate[t, h])`` in place; ``gate`` may be columns of a wider row-major matrix (its
    row stride is honoured), in the dtype of ``x``."""
    T = x.shape[0]
    if x.numel() != T * n_heads * dim or gate.dtype != x.dtype or gate.shape[0] != T or gate.shape[1] != n_heads \
            or gate.stride(1) != 1:
        raise ValueError("head_sigmoid_gate: shape/dtype mismatch")
    if not x.is_contiguous():
        raise ValueError("head_sigmoid_gate: x must be contiguous")
    _check(lib().qb_head_sigmoid_gate(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(gate.data_ptr()),
                                      int(gate.stride(0)), _code(x), T, n_heads, dim, _stream()), "head_sigmoid_gate")


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor | None, rows: torch.Tensor | None = None, store_h: bool = True) -> None:
    """``h += sum_s delta[:, s]`` (float32) and ``out = weight * h * rsqrt(mean(h^2) + eps)``.

    ``delta`` is ``[T, H]`` or ``[T, S, H]`` or None; ``rows`` (int32) selects token rows, in which case
    ``out`` has one row per entry.  ``out`` None only folds the delta into ``h``."""
    _want(h, torch.float32, "h"); _want(weight, torch.float32, "weight")
    T, H = h.shape
    S = 1
    if delta is not None:
        if delta.dim() == 3:
            S = delta.shape[1]
        if delta.shape[0] != T or delta.shape[-1] != H:
            raise ValueError("add_rmsnorm: delta shape mismatch")
    n = T if rows is None else rows.numel()
    if rows is not None:
        _want(rows, torch.int32, "rows")
    if out is not None and (out.shape[0] != n or out.shape[1] != H):
        raise ValueError("add_rmsnorm: out shape mismatch")
    if weight.numel() != H:
        raise ValueError("add_rmsnorm: weight shape mismatch")
    _check(lib().qb_add_rmsnorm(_p(h), _p(delta), _code(delta) if delta is not None else F32, S, _p(weight),
                                _p(out), _code(out) if out is not None else F32, _p(rows), n, H,
                                ctypes.c_float(eps), int(store_h), _stream()), "add_rmsnorm")


def normed_add_rmsnorm(h: torch.Tensor, y: torch.Tensor | None, y_gain: torch.Tensor | None, y_eps: float,
                       weight: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                       rows: torch.Tensor | None = None, store_h: bool = True, *, y_scale: float = 1.0,
                       y_bias: torch.Tensor | None = None, extra: torch.Tensor | None = None, extra_scale: float = 1.0,
                       extra_bias: torch.Tensor | None = None) -> None:
    """``h += y_gain * z * rsqrt(mean(z^2) + y_eps)`` (float32) and ``out = weight * h * rsqrt(mean(h^2) + eps)``: a
    sublayer's output that is normed before it joins the stream, and the norm that follows, in one launch.
    ``z = y_scale * (sum_s y[:, s] + y_bias) + extra_scale * (extra + extra_bias)``: ``y`` float32 ``[T, H]`` or
    ``[T, S, H]`` (slots added in order), ``extra`` float32 ``[T, H]`` or None, the biases ``[H]`` or None.
    ``weight`` None with ``out``: ``out`` is the stream itself (for a sublayer that reads it without a norm);
    ``y`` None: nothing joins.  ``rows`` / ``store_h`` / ``out`` None as in ``add_rmsnorm``."""
    _want(h, torch.float32, "h")
    T, H = h.shape
    S = 1
    if y is not None:
        _want(y, torch.float32, "y"); _want(y_gain, torch.float32, "y_gain")
        S = y.shape[1] if y.dim() == 3 else 1
        if y.shape[0] != T or y.shape[-1] != H or y_gain.numel() != H:
            raise ValueError("normed_add_rmsnorm: shape mismatch")
    elif extra is not None:
        raise ValueError("normed_add_rmsnorm: a second addend without a first")
    for t, n in ((y_bias, "y_bias"), (extra, "extra"), (extra_bias, "extra_bias")):
        if t is not None:
            _want(t, torch.float32, n)
            if t.shape[-1] != H or t.numel() != (T * H if n == "extra" else H):
                raise ValueError(f"normed_add_rmsnorm: {n} shape mismatch")
    n = T if rows is None else rows.numel()
    if rows is not None:
        _want(rows, torch.int32, "rows")
    if out is not None:
        if out.shape[0] != n or out.shape[1] != H:
            raise ValueError("normed_add_rmsnorm: out shape mismatch")
        if weight is not None:
            _want(weight, torch.float32, "weight")
            if weight.numel() != H:
                raise ValueError("normed_add_rmsnorm: weight shape mismatch")
    _check(lib().qb_normed_add_rmsnorm(_p(h), _p(y), S, ctypes.c_float(y_scale), _p(y_bias), _p(extra),
                                       ctypes.c_float(extra_scale), _p(extra_bias), _p(y_gain), ctypes.c_float(y_eps),
                                       _p(weight) if out is not None else ctypes.c_void_p(0), _p(out),
                                       _code(out) if out is not None else F32, _p(rows), n, H, ctypes.c_float(eps),
                                       int(store_h), _stream()), "normed_add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """``h += sum_s delta[:, s]`` in float32 (``delta`` ``[T, H]`` or ``[T, S, H]``), without a norm."""
    _want(h, torch.float32, "h")
    T, H = h.shape
    S = delta.shape[1] if delta.dim() == 3 else 1
    if delta.shape[0] != T or delta.shape[-1] != H:
        raise ValueError("residual_add: delta shape mismatch")
    _check(lib().qb_add_rmsnorm(_p(h), _p(delta), _code(delta), S, ctypes.c_void_p(0), ctypes.c_void_p(0), F32,
                                ctypes.c_void_p(0), T, H, ctypes.c_float(0.0), 1, _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    n, two_i = gate_up.shape
    if out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype:
        raise ValueError("silu_mul: shape/dtype mismatch")
    _check(lib().qb_silu_mul(_p(gate_up), _p(out), _code(out), n, two_i // 2, _stream()), "silu_mul")


def qknorm_rope_write(qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, norm_kind: int, eps: float,
                      inv_freq, pair_axis, positions, tok_pos, tok_req, block_table, nq: int, nkv: int,
                      hd: int, rd: int, page_size: int, status, *, vd: int | None = None, has_kv: bool = True,
                      q_temp_coef: float = 0.0, q_temp_every: int = 0, bias=None, v_first=None, v_lambda=None,
                      v_export=None, head_scale=None) -> None:
    """Rows ``[q | k | v | ...]`` of a fused projection (``qkv`` may be wider than the three; its row stride is
    honoured) -> normed, rotated queries in ``q_out`` and keys / values in the pages.  ``vd``: the values' head
    size when it differs from ``hd``; ``has_kv`` False: the rows start with q alone (a layer that reads another
    layer's cache); ``q_temp_every`` > 0: q is multiplied by ``1 + q_temp_coef * ln(floor((pos + 1) /
    q_temp_every) + 1)``.  ``qkv`` may hold the projection's float32 accumulators while ``q_out`` and the cache are
    bfloat16.  ``bias``: float32, added to the row's ``[q | k | v]`` first.  A per-head norm may come without gains
    (both None).  ``v_first`` (float32 ``[T, nkv * vd]``) with ``v_lambda`` (one float32 on the device): the values
    become ``(1 - lambda) v + lambda v_first`` before they are cached; ``v_export``: this layer's own values (bias
    added, not blended) are left there as float32.  ``head_scale`` (float32 ``[nq]``): a number per q head that
    multiplies the head's queries (and so its scores) after norm and rotation."""
    T = qkv.shape[0]
    vd = hd if vd is None else int(vd)
    if qkv.stride(1) != 1 or qkv.shape[1] < nq * hd + (nkv * (hd + vd) if has_kv else 0):
        raise ValueError("qknorm_rope_write: qkv width mismatch")
    if (q_out.dtype != qkv.dtype and qkv.dtype != torch.float32) or q_out.numel() != T * nq * hd:
        raise ValueError("qknorm_rope_write: q_out mismatch")
    num_pages = 0
    if k_cache is not None:
        if not has_kv:
            raise ValueError("qknorm_rope_write: rows without keys and values cannot fill a cache")
        if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
            raise ValueError("qknorm_rope_write: cache dtype differs from activations")
        if (tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or tuple(v_cache.shape[1:]) != (nkv, page_size, vd)
                or k_cache.shape[0] != v_cache.shape[0]):
            raise ValueError("qknorm_rope_write: cache shape mismatch")
        num_pages = k_cache.shape[0]
    n_row = nq * hd + (nkv * (hd + vd) if has_kv else 0)
    for t, n, size in ((bias, "bias", n_row), (v_first, "v_first", T * nkv * vd), (v_lambda, "v_lambda", 1),
                       (v_export, "v_export", T * nkv * vd), (head_scale, "head_scale", nq)):
        if t is not None:
            _want(t, torch.float32, n)
            if t.numel() != size:
                raise ValueError(f"qknorm_rope_write: {n} holds {t.numel()} numbers, {size} wanted")
    _want(inv_freq, torch.float32, "inv_freq")
    if inv_freq.numel() != rd // 2:
        raise ValueError("qknorm_rope_write: inv_freq length")
    n_axes = 1 if positions.dim() == 1 else positions.shape[1]
    for t, n in ((positions, "positions"), (tok_pos, "tok_pos"), (tok_req, "tok_req"), (block_table, "block_table")):
        _want(t, torch.int32, n)
    if pair_axis is not None:
        _want(pair_axis, torch.int32, "pair_axis")
    if norm_kind == NORM_PER_HEAD and q_norm_w is None and k_norm_w is None:
        pass                                    # every head divided by its root mean square, no gains
    elif norm_kind != NORM_NONE:
        want = (nq * hd, nkv * hd) if norm_kind == NORM_PER_LAYER else (hd, hd)
        if q_norm_w.numel() != want[0] or (has_kv and k_norm_w.numel() != want[1]):
            raise ValueError("qknorm_rope_write: norm weight length does not fit the norm kind")
    _check(lib().qb_qknorm_rope_write(
        ctypes.c_void_p(qkv.data_ptr()), _code(qkv), _code(q_out), int(qkv.stride(0)), _p(q_out), _p(k_cache), _p(v_cache),
        _p(q_norm_w), _p(k_norm_w) if has_kv else ctypes.c_void_p(0), norm_kind,
        ctypes.c_float(eps), _p(inv_freq), _p(pair_axis), _p(positions), n_axes, _p(tok_pos), _p(tok_req),
        _p(block_table), block_table.shape[1], T, nq, nkv, hd, vd, int(has_kv), rd, ctypes.c_float(q_temp_coef),
        int(q_temp_every), page_size, num_pages, _p(bias), _p(v_first), _p(v_lambda), _p(v_export), _p(head_scale),
        _p(status), _stream()), "qknorm_rope_write")


def paged_attention_simt(q, k_cache, v_cache, out, tok_pos, tok_req, block_table, scale: float,
                         window: int, status) -> None:
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    vd = v_cache.shape[3]
    if (hd2 != hd or tuple(out.shape) != (T, nq, vd) or out.dtype != q.dtype or k_cache.dtype != q.dtype
            or v_cache.dtype != q.dtype or tuple(v_cache.shape[:3]) != (num_pages, nkv, page_size)):
        raise ValueError("paged_attention: shape/dtype mismatch")
    _check(lib().qb_paged_attention_simt(
        _p(q), _code(q), _p(k_cache), _p(v_cache), _p(out), _p(tok_pos), _p(tok_req), _p(block_table),
        block_table.shape[1], T, nq, nkv, hd, vd, page_size, num_pages, ctypes.c_float(scale), int(window),
        _p(status), _stream()), "paged_attention_simt")


def attn_span_rows(hd: int, nq: int, nkv: int, page_size: int) -> int:
    """Query rows (token x head-of-group) per tile of the kernel that runs portions of these shapes."""
    return int(lib().qb_attn_span_rows(int(hd), int(nq), int(nkv), int(page_size)))


def attn_decode_parts(nkv: int, max_len: int) -> int:
    """Entries per (token, q head) row of the decode attention scratch for contexts of up to ``max_len`` keys."""
    n = int(lib().qb_attn_decode_parts(int(nkv), int(max_len)))
    if n < 2:
        raise KernelError(f"attn_decode_parts({nkv}, {max_len}) failed with code {n}")
    return n


ATTN_DECODE_MAX_GROUP = 64      # q heads per kv head that the decode kernel takes


def attn_span_tc_supported(nq: int, nkv: int, hd: int, page_size: int) -> bool:
    """Whether portions of these shapes run on the tcgen05 kernel (else on the mma.sync kernel)."""
    return bool(lib().qb_attn_span_tc_supported(int(nq), int(nkv), int(hd), int(page_size)))


def attn_span(q, k_cache, v_cache, out, tok_pos, block_table, tiles, scale: float, window: int, status) -> None:
    """bfloat16 tensor-core attention for prompt portions.  ``tiles`` int32 [n, 4]: request row, first
    token row of the portion, tokens in the portion, first flattened (token*G + head) row of the tile."""
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    _want(q, torch.bfloat16, "q"); _want(k_cache, torch.bfloat16, "k_cache"); _want(tiles, torch.int32, "tiles")
    if hd2 != hd or out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError("attn_span: shape/dtype mismatch")
    _check(lib().qb_attn_span(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(tok_pos), _p(block_table),
                              block_table.shape[1], _p(tiles), tiles.shape[0], nq, nkv, hd, page_size, num_pages,
                              ctypes.c_float(scale), int(window), _p(status), _stream()), "attn_span")


def attn_decode(q, k_cache, v_cache, out, part_o, part_ml, dec_tok, n_dec: int, tok_pos, tok_req, block_table,
                scale: float, window: int, n_parts: int, status) -> None:
    """bfloat16 tensor-core attention for single tokens; ``part_o`` / ``part_ml`` are float32 scratch of
    at least n_dec*nq*n_parts*hd and n_dec*nq*n_parts*2 elements, ``n_parts`` from ``attn_decode_parts``."""
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    _want(q, torch.bfloat16, "q"); _want(k_cache, torch.bfloat16, "k_cache")
    _want(part_o, torch.float32, "part_o"); _want(part_ml, torch.float32, "part_ml"); _want(dec_tok, torch.int32, "dec_tok")
    if hd2 != hd or out.shape != q.shape or out.dtype != q.dtype:
        raise ValueError("attn_decode: shape/dtype mismatch")
    if part_o.numel() < n_dec * nq * n_parts * hd or part_ml.numel() < n_dec * nq * n_parts * 2:
        raise ValueError("attn_decode: scratch too small")
    _check(lib().qb_attn_decode(_p(q), _p(k_cache), _p(v_cache), _p(out), _p(part_o), _p(part_ml), _p(dec_tok),
                                int(n_dec), _p(tok_pos), _p(tok_req), _p(block_table), block_table.shape[1], nq, nkv,
                                hd, page_size, num_pages, ctypes.c_float(scale), int(window), int(n_parts),
                                _p(status), _stream()), "attn_decode", 2)


def split3_bf16(w: torch.Tensor) -> torch.Tensor:
    """A float32 tensor as three bfloat16 tensors ``[3, *w.shape]`` whose sum is ``w`` to float32 accuracy
    (each is the bfloat16 rounding of what the ones before leave over)."""
    _want(w, torch.float32, "w")
    w = w.contiguous()
    out = torch.empty((3, *w.shape), dtype=torch.bfloat16, device=w.device)
    _check(lib().qb_split3_bf16(_p(w), _p(out), ctypes.c_longlong(w.numel()), _stream()), "split3_bf16")
    return out


def router_gemm_mma_parts(K: int) -> int:
    """Ranges the inner dimension of ``router_gemm_mma`` is cut into (a function of K alone)."""
    return int(lib().qb_router_gemm_mma_parts(int(K)))


def router_gemm_mma(x: torch.Tensor, pieces: torch.Tensor, logits: torch.Tensor) -> None:
    """``sum_p logits[p, T, E] = x[T, K] @ (pieces[0] + pieces[1] + pieces[2]).T`` in float32 on the tensor
    cores, ``pieces`` from ``split3_bf16`` of the float32 gate; the inner dimension in fixed chunks of 64,
    and in ``router_gemm_mma_parts(K)`` fixed ranges whose sums ``router_topk`` adds in order."""
    T, K = x.shape
    _want(x, torch.bfloat16, "x"); _want(pieces, torch.bfloat16, "pieces"); _want(logits, torch.float32, "logits")
    E = pieces.shape[1]
    parts = router_gemm_mma_parts(K)
    if (pieces.shape[0] != 3 or pieces.shape[2] != K or logits.numel() != parts * T * E
            or not logits.is_contiguous()):
        raise ValueError(f"router_gemm_mma: shape mismatch (logits must be [{parts}, {T}, {E}])")
    _check(lib().qb_router_gemm_mma(_p(x), _p(pieces), _p(logits), T, E, K, _stream()), "router_gemm_mma")


ROUTE_SIGMOID_RAW, ROUTE_SIGMOID_RENORM, ROUTE_SOFTMAX_CHOSEN, ROUTE_SOFTMAX_ALL = 0, 1, 2, 3


def router_topk(logits, bias, idx_out, w_out, renorm, scale: float) -> None:
    """``logits`` [T, E], or [P, T, E] partial sums that are added in index order first.  ``renorm``: False / True
    (sigmoid scores as they are / divided by their sum; the bias enters the choice only), or
    ``ROUTE_SOFTMAX_CHOSEN``: the choice is by ``logit + bias`` and the weights are the softmax over the chosen
    values, or ``ROUTE_SOFTMAX_ALL``: the scores are the softmax over all logits, the choice is by ``score + bias``
    and the weights are the chosen scores as they are."""
    _want(logits, torch.float32, "logits"); _want(idx_out, torch.int32, "idx_out"); _want(w_out, torch.float32, "w_out")
    n_partials = 1 if logits.dim() == 2 else logits.shape[0]
    T, E = logits.shape[-2:]
    k = idx_out.shape[1]
    if bias is not None:
        _want(bias, torch.float32, "bias")
    _check(lib().qb_router_topk(_p(logits), n_partials, _p(bias), _p(idx_out), _p(w_out), T, E, k, int(renorm),
                                ctypes.c_float(scale), _stream()), "router_topk")


ROUTER_SMALL_MAX_TILE_BYTES = 200 * 1024          # eight token rows must fit the router's shared-memory tile


def router_small_selects(n_tokens: int, n_experts: int, top_k: int) -> bool:
    """Whether ``router_small`` can select and lay the expert plan down in the same launch."""
    return bool(lib().qb_router_small_selects(int(n_tokens), int(n_experts), int(top_k)))


def router_small(x, gate, bias, logits, idx_out=None, w_out=None, renorm: bool = True, scale: float = 1.0, *,
                 counters=None, bm: int = 0, plan=None, sorted_pair=None, tile_expert=None, tile_row0=None,
                 status=None, tiled_experts: int = 0) -> None:
    """Float32 router logits ``logits[T, E] = x[T, K] @ gate[E, K].T`` on the CUDA cores, every logit one sum in
    an order that depends on K alone.  With ``idx_out`` / ``w_out`` / the plan tensors (and
    ``router_small_selects``): the selection (``router_topk``) and the expert plan (``moe_plan``) in the same
    launch; ``counters``: ``1 + ceil(T / 8)`` int32 that are zero before the call and are left zero.
    ``tiled_experts`` > 0: only the first so many experts get tiles in the plan (the others have no weights)."""
    _want(gate, torch.float32, "gate"); _want(logits, torch.float32, "logits")
    T, K = x.shape
    E = gate.shape[0]
    if gate.shape[1] != K or tuple(logits.shape) != (T, E):
        raise ValueError("router_small: shape mismatch")
    if 8 * K * x.element_size() > ROUTER_SMALL_MAX_TILE_BYTES:
        raise ValueError(f"router_small: rows of {K} elements do not fit the kernel's shared-memory tile "
                         f"(at most {ROUTER_SMALL_MAX_TILE_BYTES // (8 * x.element_size())})")
    if bias is not None:
        _want(bias, torch.float32, "bias")
    select = idx_out is not None
    k = 0
    if select:
        _want(idx_out, torch.int32, "idx_out"); _want(w_out, torch.float32, "w_out"); _want(counters, torch.int32, "counters")
        k = idx_out.shape[1]
        if not router_small_selects(T, E, k) or counters.numel() < 1 + -(-T // 8):
            raise ValueError("router_small: sizes outside what the selecting form takes, or too few counters")
    _check(lib().qb_router_small(_p(x), _code(x), _p(gate), _p(bias), _p(logits), _p(idx_out), _p(w_out), T, E, K, k,
                                 int(renorm), ctypes.c_float(scale), int(select), _p(counters), int(bm), _p(plan),
                                 _p(sorted_pair), _p(tile_expert), _p(tile_row0),
                                 tile_expert.numel() if tile_expert is not None else 0, _p(status), int(tiled_experts),
                                 _stream()), "router_small")


MOE_SIMT_BM = 32


def moe_plan_sizes(n_pairs: int, n_experts: int, bm: int) -> tuple[int, int]:
    """(plan words, max tiles) for ``n_pairs`` (token, slot) pairs."""
    return 4 * n_experts + 4, (n_pairs + bm - 1) // bm + min(n_experts, n_pairs)


def moe_plan(idx, n_experts: int, bm: int, plan, sorted_pair, tile_expert, tile_row0, status, tiled_experts: int = 0) -> None:
    """``tiled_experts`` > 0: only the first so many experts get tiles (the others have no weights; their pairs are
    still counted and sorted)."""
    n_pairs = idx.numel()
    max_tiles = tile_expert.numel()
    _check(lib().qb_moe_plan(_p(idx), n_pairs, n_experts, bm, _p(plan), _p(sorted_pair), _p(tile_expert),
                             _p(tile_row0), max_tiles, _p(status), int(tiled_experts), _stream()), "moe_plan", 3)


def identity_slots(x, idx, w, y, first_identity: int) -> None:
    """``y[t, j] = w[t, j] * x[t]`` for every choice ``idx[t, j] >= first_identity`` (experts that hand their input
    through); the other slots are left alone.  ``y`` float32 ``[T, k, H]``."""
    _want(idx, torch.int32, "idx"); _want(w, torch.float32, "w"); _want(y, torch.float32, "y")
    T, k, H = y.shape
    if tuple(x.shape) != (T, H) or idx.numel() != T * k or w.numel() != T * k:
        raise ValueError("identity_slots: shape mismatch")
    _check(lib().qb_identity_slots(_p(x), _code(x), _p(idx), _p(w), _p(y), T * k, k, H, int(first_identity), _stream()),
           "identity_slots")


EXPERT_ACT_SILU, EXPERT_ACT_CLAMPED = 0, 1


def moe_grouped_simt(mode: int, x, weights, out, sorted_pair, pair_w, plan, tile_expert, tile_row0,
                     n_experts: int, top_k: int, act: tuple = (0, 0.0, 1.0)) -> None:
    """mode 1: ``out[p, :I] = silu(x[tok] W13_e[:I]^T) * (x[tok] W13_e[I:]^T)``; mode 2:
    ``out[pair] = w[pair] * (x[p] W2_e^T)``; mode 3: ``out[p] = relu(x[tok] W1_e^T)^2`` (ungated experts);
    rows p sorted by expert (see ``moe_plan``).  ``weights`` may hold fewer experts than the plan counts when the
    plan gives the others no tiles.  ``act`` = (kind, limit, alpha) for mode 1: ``EXPERT_ACT_CLAMPED`` multiplies both
    products by the pair's routing weight first (the expert reads ``w * x``), then ``g = min(gate, limit)``,
    ``u = clamp(up, -limit, limit)``, ``g * sigmoid(alpha g) * (u + 1)``.  Mode 2 with ``pair_w`` None: no weights."""
    K = x.shape[1]
    N = out.shape[1]
    want = (2 * N, K) if mode == 1 else (N, K)
    if tuple(weights.shape[1:]) != want or not 0 < weights.shape[0] <= n_experts:
        raise ValueError(f"moe_grouped: weights {tuple(weights.shape)} do not fit {n_experts} experts of {want}")
    _check(lib().qb_moe_grouped_simt(mode, _p(x), _code(x), _p(weights), _code(weights), _p(out), _code(out),
                                     _p(sorted_pair), _p(pair_w), _p(plan), _p(tile_expert), _p(tile_row0),
                                     tile_expert.numel(), n_experts, top_k, K, N, int(act[0]), ctypes.c_float(act[1]),
                                     ctypes.c_float(act[2]), _stream()), "moe_grouped_simt")


def expert_gemm_tc_supported(x: torch.Tensor, hidden: int, inner: int) -> bool:
    """The tcgen05 expert kernel takes bfloat16 and inner dimensions that are multiples of 8 (16-byte rows
    for TMA)."""
    return x.dtype == torch.bfloat16 and hidden % 8 == 0 and inner % 8 == 0


def expert_tile_rows(n_tokens: int, rows_per_expert: float = 0.0) -> int:
    """Token tile (the MMA's N) of the tcgen05 expert kernel for a step of ``n_tokens`` tokens: an expert
    never receives more rows than there are tokens; from about a hundred rows an expert on average
    (``rows_per_expert``) the products are no longer bound by memory alone, and tiles of 256 rows, which pairs
    of blocks take, read the operands least often (measured on a B200, both products of a layer: 96 rows an
    expert 1,464 against 1,399 us with tiles of 128; 128 rows 1,559 against 1,755 us; 256 rows 2,372 against
    2,889 us; an expert's last tile of a few rows costs the tensor cores only those rows)."""
    for nt in (16, 32, 64):
        if n_tokens <= nt:
            return nt
    big = int(os.environ.get("QUANTA_B200_EXPERT_TILE", "0"))
    if big:
        return big
    return 256 if rows_per_expert >= 112 else 128


def gather_rows(x, out, sorted_pair, top_k: int) -> None:
    """``out[p] = x[sorted_pair[p] // top_k]``: the token rows in expert order, contiguous for TMA."""
    n_pairs, K = out.shape
    _want(x, torch.bfloat16, "x"); _want(out, torch.bfloat16, "out")
    if x.shape[1] != K or sorted_pair.numel() != n_pairs:
        raise ValueError("gather_rows: shape mismatch")
    _check(lib().qb_gather_rows(_p(x), _p(out), _p(sorted_pair), n_pairs, top_k, K, _stream()), "gather_rows")


def expert_gemm_tc(mode: int, x_rows, weights, out, sorted_pair, pair_w, plan, tile_expert, tile_row0,
                   n_experts: int, tile_rows: int, status, gather_top_k: int = 0, weight_experts: int = 0,
                   act: tuple = (0, 0.0, 1.0)) -> None:
    """Expert products on tcgen05/TMEM fed by TMA.  ``x_rows`` bf16 [pairs, K] in expert order; mode 1:
    ``out[p, :I] = silu(gate) * up`` (bf16), mode 2: ``out[pair(p)] = w[pair(p)] * down`` (float32), mode 3:
    ``out[p] = relu(up)^2`` (bf16; ungated experts, weights ``[E, I, K]``).  The plan's
    tile list must have been made with ``bm = tile_rows``.  Mode 1 or 3 with ``gather_top_k`` > 0: ``x_rows`` is the
    step's activations [T, K] and the kernel fetches the row of token ``pair // gather_top_k`` itself, one
    TMA box a row (for steps of few tokens: it saves the gathered copy and its launch).  ``weight_experts`` > 0: the
    plan counts ``n_experts`` experts of which only the first so many have weights (and tiles).  ``act`` and a
    ``pair_w`` of None in mode 2 as in ``moe_grouped_simt``."""
    n_x, K = x_rows.shape
    n_pairs = sorted_pair.numel()
    N = out.shape[1]
    n_w = weight_experts or n_experts
    want = (n_w, 2 * N, K) if mode == 1 else (n_w, N, K)
    if tuple(weights.shape) != want:
        raise ValueError(f"expert_gemm_tc: weights {tuple(weights.shape)} != {want}")
    if gather_top_k == 0 and n_x != n_pairs:
        raise ValueError(f"expert_gemm_tc: {n_x} rows for {n_pairs} pairs")
    _want(x_rows, torch.bfloat16, "x_rows"); _want(weights, torch.bfloat16, "weights")
    _want(out, torch.float32 if mode == 2 else torch.bfloat16, "out")
    _check(lib().qb_expert_gemm_tc(mode, _p(x_rows), _p(weights), _p(out), _p(sorted_pair), _p(pair_w), _p(plan),
                                   _p(tile_expert), _p(tile_row0), tile_expert.numel(), n_pairs, n_experts, K, N,
                                   int(tile_rows), int(gather_top_k), n_x, _p(status), int(weight_experts), int(act[0]),
                                   ctypes.c_float(act[1]), ctypes.c_float(act[2]), _stream()),
           "expert_gemm_tc")


# ---- state slots (csrc/request_state.h) ------------------------------------------------------------------
SLOT_WORDS = 16
SLOT_LIVE, SLOT_POSITION, SLOT_PROMPT, SLOT_DRAWN, SLOT_LAST, SLOT_SEED_LO, SLOT_SEED_HI, SLOT_TOP_K = range(8)
SLOT_TEMPERATURE, SLOT_TOP_P, SLOT_MIN_P = 8, 9, 10


def slot_record(*, position: int = 0, prompt_len: int = 0, drawn: int = 0, last: int = 0, seed: int = 0,
                temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0) -> torch.Tensor:
    """A live request's record as int32 ``[SLOT_WORDS]`` on the host (floats as their bit patterns)."""
    import struct

    def bits(x: float) -> int:
        return struct.unpack("<i", struct.pack("<f", float(x)))[0]

    def word(x: int) -> int:
        x &= 0xFFFFFFFF
        return x - (1 << 32) if x >= (1 << 31) else x

    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    rec = [0] * SLOT_WORDS
    rec[SLOT_LIVE], rec[SLOT_POSITION], rec[SLOT_PROMPT], rec[SLOT_DRAWN], rec[SLOT_LAST] = 1, position, prompt_len, drawn, last
    rec[SLOT_SEED_LO], rec[SLOT_SEED_HI], rec[SLOT_TOP_K] = word(seed), word(seed >> 32), int(top_k)
    rec[SLOT_TEMPERATURE], rec[SLOT_TOP_P], rec[SLOT_MIN_P] = bits(temperature), bits(top_p), bits(min_p)
    return torch.tensor(rec, dtype=torch.int32)


def slots_advance(slots, req_slot, req_start, req_len_after, n_requests: int, status) -> None:
    """Move each request's position in its state slot to what it holds after the step; a slot that is free
    or at another position than the step assumes is recorded in ``status``."""
    _want(slots, torch.int32, "slots")
    if slots.dim() != 2 or slots.shape[1] != SLOT_WORDS:
        raise ValueError(f"slots must be [n, {SLOT_WORDS}]")
    _check(lib().qb_slots_advance(_p(slots), slots.shape[0], _p(req_slot), _p(req_start), _p(req_len_after),
                                  int(n_requests), _p(status), _stream()), "slots_advance")


def sample_rows(logits, slots, row_slot, out, all_greedy: bool = False) -> None:
    """One token a row of float32 logits.  ``slots`` int32 ``[n_slots, SLOT_WORDS]`` and ``row_slot`` int32
    ``[n]``: each row's options and draw number come from its slot's record, which then counts the draw and
    holds the token.  ``slots`` None: every row is greedy (first maximum) and nothing is recorded.
    ``all_greedy``: the caller knows every row's temperature is <= 0 (a large vocabulary is then cut over
    many blocks)."""
    _want(logits, torch.float32, "logits"); _want(out, torch.int32, "out")
    n, V = logits.shape
    n_slots = 0
    if slots is not None:
        _want(slots, torch.int32, "slots"); _want(row_slot, torch.int32, "row_slot")
        if slots.dim() != 2 or slots.shape[1] != SLOT_WORDS or row_slot.numel() != n:
            raise ValueError("sample_rows: slots must be [n_slots, SLOT_WORDS] and row_slot [n]")
        n_slots = slots.shape[0]
    if (slots is None or all_greedy) and V >= 4096:
        # all greedy: a row is cut over many blocks, then the first maximum of the chunks is taken
        parts = 32
        sv = torch.empty(n * parts, dtype=torch.float32, device=logits.device)
        si = torch.empty(n * parts, dtype=torch.int32, device=logits.device)
        _check(lib().qb_argmax_rows(_p(logits), n, V, parts, _p(sv), _p(si), _p(slots), _p(row_slot), n_slots, _p(out),
                                    _stream()), "argmax_rows", 2)
        return
    _check(lib().qb_sample_rows(_p(logits), n, V, _p(slots), _p(row_slot), n_slots, _p(out), _stream()), "sample_rows")


def apply_penalties(logits, prev, prev_off, pparams) -> None:
    _want(logits, torch.float32, "logits")
    n, V = logits.shape
    _check(lib().qb_apply_penalties(_p(logits), n, V, _p(prev), _p(prev_off), _p(pparams), _stream()),
           "apply_penalties")


# ---- short convolution, delta-rule recurrence, latent attention ---------------------------------------
def short_conv(x, weight, state, out, tok_req, req_start, req_slot, *, bias=None, silu: bool = False,
               plain: bool = False) -> None:
    """``out[t] = x[t] + sum_j weight[:, j] * x[t - taps + 1 + j]`` over each request's own rows, the rows
    before a portion taken from ``state`` ``[slots, taps - 1, C]`` (float32, newest last), which then holds
    the request's last ``taps - 1`` inputs.  ``x`` float32 ``[T, C]`` (a column range of wider rows is fine),
    ``weight`` float32 ``[C, taps]``.  ``silu``: ``out[t] = silu(bias + sum_j ...)`` instead, the input not added back; ``plain``: the sum alone."""
    _want(x, torch.float32, "x"); _want(weight, torch.float32, "weight"); _want(state, torch.float32, "state")
    T, C = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != C or tuple(out.shape) != (T, C) or tuple(state.shape[1:]) != (max(taps - 1, 0), C):
        raise ValueError("short_conv: shape mismatch")
    if x.stride(1) != 1 or not weight.is_contiguous() or not out.is_contiguous() or not state.is_contiguous():
        raise ValueError("short_conv: rows must be contiguous")
    if bias is not None:
        _want(bias, torch.float32, "bias")
        if bias.numel() != C or not silu:
            raise ValueError("short_conv: the bias has C numbers and belongs to the silu form")
    if silu and plain:
        raise ValueError("short_conv: silu or the sum alone, not both")
    R = req_slot.numel()
    _check(lib().qb_short_conv(ctypes.c_void_p(x.data_ptr()), _p(weight), _p(state), _p(out), _code(out), _p(tok_req),
                               _p(req_start), _p(req_slot), T, R, C, taps, int(x.stride(0)), _p(bias),
                               2 if plain else int(silu), _stream()), "short_conv",
           2 if taps > 1 and not lib().qb_short_conv_one_launch(T, R) else 1)


DELTA_RULE_MAX_DIM = 256


def delta_rule(proj, offsets, wpre, a_bias, w_bias, state, out, req_start, req_slot, n_heads: int, dim: int,
               decay_scale: float, unit_eps: float) -> None:
    """The recurrence ``S <- diag(w) S - (a u)(u^T S) + k v^T``, ``o = S^T r`` per (request, head) over the
    step's tokens, from and into ``state`` ``[slots, heads, dim, dim]`` float32.  ``proj`` float32 ``[T, P]``
    holds r, k, v and the pre-activation of a at the column ``offsets`` (r, k, v, a), heads x dim each;
    ``wpre`` float32 ``[T, heads*dim]`` the pre-activation of the decay; ``out`` float32 ``[T, heads, dim]``."""
    for t, n in ((proj, "proj"), (wpre, "wpre"), (a_bias, "a_bias"), (w_bias, "w_bias"), (state, "state"), (out, "out")):
        _want(t, torch.float32, n)
    T = proj.shape[0]
    HD = n_heads * dim
    if (tuple(wpre.shape) != (T, HD) or out.numel() != T * HD or a_bias.numel() != HD or w_bias.numel() != HD
            or tuple(state.shape[1:]) != (n_heads, dim, dim) or any(o < 0 or o + HD > proj.shape[1] for o in offsets)):
        raise ValueError("delta_rule: shape mismatch")
    if proj.stride(1) != 1:
        raise ValueError("delta_rule: proj rows must be dense")
    r_off, k_off, v_off, a_off = (int(o) for o in offsets)
    R = req_slot.numel()
    scratch = torch.empty(3 * T * HD, dtype=torch.float32, device=proj.device)      # w, a*u, u of every (token, head)
    _check(lib().qb_delta_rule(ctypes.c_void_p(proj.data_ptr()), int(proj.stride(0)), r_off, k_off, v_off, a_off,
                               _p(wpre), _p(a_bias), _p(w_bias), _p(state), _p(out), _p(scratch), _p(req_start),
                               _p(req_slot), R, T, n_heads, dim, ctypes.c_float(decay_scale), ctypes.c_float(unit_eps),
                               _stream()), "delta_rule", 2)


def head_norm_gate(o, proj, gate_off: int, gain, out, n_heads: int, dim: int, eps: float, gate: str = "sigmoid") -> None:
    """``out[t, h] = o[t, h] / rms(o[t, h]) * gain * act(proj[t, gate_off + h*dim ...])``; ``gain`` has
    ``n_heads * dim`` elements, or ``dim`` that every head shares; ``gate``: ``"sigmoid"`` or ``"silu"``."""
    _want(o, torch.float32, "o"); _want(proj, torch.float32, "proj"); _want(gain, torch.float32, "gain")
    T = proj.shape[0]
    if o.numel() != T * n_heads * dim or tuple(out.shape) != (T, n_heads * dim) or gain.numel() not in (n_heads * dim, dim):
        raise ValueError("head_norm_gate: shape mismatch")
    if gate not in ("sigmoid", "silu"):
        raise ValueError(f"head_norm_gate: gate {gate!r} is not 'sigmoid' or 'silu'")
    shared = int(gain.numel() == dim and n_heads > 1)
    gate_ptr = ctypes.c_void_p(proj.data_ptr() + 4 * int(gate_off))
    _check(lib().qb_head_norm_gate(_p(o), gate_ptr, int(proj.stride(0)), _p(gain), _p(out), _code(out), T, n_heads, dim,
                                   ctypes.c_float(eps), shared, int(gate == "silu"), _stream()), "head_norm_gate")


GLA_MAX_DIM = 256


def gla(proj, offsets, inner_off: int, rank: int, w2, bias, state, out, req_start, req_slot, n_heads: int, dim: int,
        vdim: int, tau: float, q_scale: float, segments: bool | None = None) -> None:
    """Gated linear attention ``S <- diag(alpha) S + k v^T``, ``o = q_scale * S^T q`` per (request, head) over the
    step's tokens, from and into ``state`` ``[slots, heads, dim, vdim]`` float32.  ``proj`` float32 ``[T, P]`` holds
    q, k (heads x dim) and v (heads x vdim) at the column ``offsets`` (q, k, v) and the ``rank`` inner values of
    the decay at ``inner_off``; ``alpha = sigmoid(w2 inner + bias) ^ (1 / tau)`` with ``w2`` ``[heads*dim, rank]``
    and ``bias`` float32; ``out`` float32 ``[T, heads, vdim]``.  ``segments`` False keeps a step with long
    portions on the one chain in time (else such steps run as segments in three passes)."""
    for t, n in ((proj, "proj"), (bias, "bias"), (state, "state"), (out, "out")):
        _want(t, torch.float32, n)
    T = proj.shape[0]
    HD, HE = n_heads * dim, n_heads * vdim
    q_off, k_off, v_off = (int(o) for o in offsets)
    if (out.numel() != T * HE or bias.numel() != HD or tuple(w2.shape) != (HD, rank)
            or tuple(state.shape[1:]) != (n_heads, dim, vdim) or proj.stride(1) != 1
            or any(o < 0 or o + n > proj.shape[1] for o, n in ((q_off, HD), (k_off, HD), (v_off, HE), (inner_off, rank)))):
        raise ValueError("gla: shape mismatch")
    R = req_slot.numel()
    scratch = torch.empty(T * HD, dtype=torch.float32, device=proj.device)      # alpha of every (token, channel)
    # steps with long portions run as segments in three passes (see the kernel file); they need room for a state
    # per segment
    fn = lib().qb_gla_segment_scratch
    fn.restype = ctypes.c_longlong
    n_seg_floats = int(fn(R, T, n_heads, dim, vdim)) if segments is not False else 0
    seg_scratch = torch.empty(n_seg_floats, dtype=torch.float32, device=proj.device) if n_seg_floats else None
    _check(lib().qb_gla(ctypes.c_void_p(proj.data_ptr()), int(proj.stride(0)), q_off, k_off, v_off, int(inner_off),
                        int(rank), _p(w2), _code(w2), _p(bias), _p(state), _p(out), _p(scratch), _p(seg_scratch),
                        _p(req_start), _p(req_slot), R, T, n_heads, dim, vdim, ctypes.c_float(tau),
                        ctypes.c_float(q_scale), _stream()), "gla", 5 if n_seg_floats else 2)


def tanh_cols(x, off: int, n: int, out) -> None:
    """``out[t, :n] = tanh(x[t, off : off + n])`` in the dtype of ``out``."""
    _want(x, torch.float32, "x")
    T = x.shape[0]
    if tuple(out.shape) != (T, n) or off + n > x.shape[1]:
        raise ValueError("tanh_cols: shape mismatch")
    _check(lib().qb_tanh_cols(ctypes.c_void_p(x.data_ptr()), int(x.stride(0)), int(off), _p(out), _code(out), T, n,
                              _stream()), "tanh_cols")


LATENT_MAX_RANK = 512


def latent_write(dkv, gain, inv_freq, cache, tok_pos, tok_req, block_table, rank: int, rot: int, rotated: int,
                 page_size: int, eps: float, status) -> None:
    """Rows ``[T, rank + rot]`` float32 -> the cache rows of their positions: RMS norm with ``gain`` of the
    first ``rank``, rotation by the position of the first ``rotated`` of the last ``rot``.  ``cache`` ``[pages, 1, page_size, rank + rot]``."""
    _want(dkv, torch.float32, "dkv"); _want(gain, torch.float32, "gain"); _want(inv_freq, torch.float32, "inv_freq")
    T = dkv.shape[0]
    if (dkv.shape[1] != rank + rot or gain.numel() != rank or inv_freq.numel() != rotated // 2
            or tuple(cache.shape[1:]) != (1, page_size, rank + rot)):
        raise ValueError("latent_write: shape mismatch")
    _check(lib().qb_latent_write(_p(dkv), _p(gain), _p(inv_freq), _p(cache), _code(cache), _p(tok_pos), _p(tok_req),
                                 _p(block_table), block_table.shape[1], T, rank, rot, int(rotated), page_size,
                                 cache.shape[0], ctypes.c_float(eps), _p(status), _stream()), "latent_write")


def latent_query(q, inv_freq, q_plain, q_rot, tok_pos, n_heads: int, dim: int, rot: int, rotated: int) -> None:
    """``q`` float32 ``[T, heads, dim + rot]`` -> ``q_plain`` ``[heads, T, dim]`` and ``q_rot`` float32
    ``[T, heads, rot]``, its first ``rotated`` dimensions rotated by the position."""
    _want(q, torch.float32, "q"); _want(q_rot, torch.float32, "q_rot")
    T = q.shape[0]
    if q.numel() != T * n_heads * (dim + rot) or q_plain.numel() != T * n_heads * dim or q_rot.numel() != T * n_heads * rot:
        raise ValueError("latent_query: shape mismatch")
    _check(lib().qb_latent_query(_p(q), _p(inv_freq), _p(q_plain), _code(q_plain), _p(q_rot), _p(tok_pos), T, n_heads,
                                 dim, rot, int(rotated), _stream()), "latent_query")


def latent_attend_uses_tensor_cores(cache_dtype, rank: int, rot: int) -> bool:
    """Whether ``latent_attend`` runs these shapes on the tensor cores (bfloat16 cache, rank 64/128/256/512, rot a
    multiple of 16) or on the CUDA cores (float32 arithmetic; every other shape, and the float32 path)."""
    return cache_dtype == torch.bfloat16 and bool(lib().qb_latent_attend_mma_supported(int(rank), int(rot)))


LATENT_MMA_ROWS = 32        # (token, head) rows a block of the tensor-core kernel takes


def latent_attend(q_lat, q_rot, cache, sink, out, tok_pos, tok_req, block_table, scale: float, n_ranges: int,
                  status, req_start=None, tensor_cores: bool | None = None) -> None:
    """Causal softmax attention of every token and head over the cached latent rows, with an optional sink.
    ``q_lat`` ``[heads, T, rank]``, ``q_rot`` float32 ``[T, heads, rot]``, ``out`` ``[heads, T, rank]``; each
    token's keys are cut into ``n_ranges`` ranges that run as blocks of their own and are merged in order.
    With ``req_start`` (int32 ``[requests + 1]``, the step's token rows of each request; token ``t`` belongs to
    request ``tok_req[t]``) and shapes that ``latent_attend_uses_tensor_cores`` takes, the scores and sums run on
    the tensor cores; ``tensor_cores`` False keeps them on the CUDA cores."""
    H, T, C = q_lat.shape
    num_pages, one, page_size, W = cache.shape
    R = W - C
    if one != 1 or q_rot.numel() != T * H * R or tuple(out.shape) != (H, T, C) or out.dtype != cache.dtype:
        raise ValueError("latent_attend: shape/dtype mismatch")
    if sink is not None:
        _want(sink, torch.float32, "sink")
    part = torch.empty(T * H * n_ranges * (C + 2), dtype=torch.float32, device=q_lat.device)
    mma = (req_start is not None and q_lat.dtype == torch.float32 and tensor_cores is not False
           and latent_attend_uses_tensor_cores(cache.dtype, C, R))
    if tensor_cores and not mma:
        raise ValueError("latent_attend: these shapes or dtypes do not run on the tensor cores")
    if mma:
        n_req = req_start.numel() - 1
        max_tiles = -(-T * H // LATENT_MMA_ROWS) + n_req
        _check(lib().qb_latent_attend_mma(_p(q_lat), _p(q_rot), _p(cache), _p(part), _p(tok_pos), _p(req_start),
                                          _p(block_table), block_table.shape[1], n_req, T, H, C, R, page_size, num_pages,
                                          int(n_ranges), max_tiles, ctypes.c_float(scale), _p(status), _stream()),
               "latent_attend_mma")
    else:
        _check(lib().qb_latent_attend(_p(q_lat), _code(q_lat), _p(q_rot), _p(cache), _code(cache), _p(part), _p(tok_pos),
                                      _p(tok_req), _p(block_table), block_table.shape[1], T, H, C, R, page_size,
                                      num_pages, int(n_ranges), ctypes.c_float(scale), _p(status), _stream()),
               "latent_attend")
    _check(lib().qb_latent_merge(_p(part), _p(sink), _p(out), _code(out), T, H, C, int(n_ranges), _stream()),
           "latent_merge")


# ---- sliding-window attention with extras (csrc/window_attention.cu) ---------------------------------------------
def window_attention_uses_tensor_cores(dtype, hd: int, vd: int) -> bool:
    """Whether ``window_attention`` can run these shapes on the tensor cores (bfloat16, key sizes that are multiples
    of 16 up to 256, value sizes that are multiples of 16 up to 128)."""
    return dtype == torch.bfloat16 and bool(lib().qb_window_attention_mma_supported(BF16, int(hd), int(vd)))


def window_attention(q, k_cache, v_cache, out, tok_pos, tok_req, block_table, scale: float, window: int, status, *,
                     dist_bias=None, sink=None, softcap: float = 0.0, pool: int = 0, pooled_k=None, pooled_v=None,
                     pool_table=None, talk=None, scratch=None, n_split: int | None = None, n_requests: int | None = None,
                     tensor_cores: bool | None = None) -> None:
    """Softmax attention of every token over the last ``window`` keys of its request (0: all of them).  Options:
    ``dist_bias`` float32 ``[window, heads]`` added to the score by distance; ``sink`` float32 ``[heads]``, a term
    ``exp(sink)`` of the denominator; ``softcap`` c > 0: ``score <- c tanh(score / c)``; ``pool`` P with the pooled
    pages and their block table: one more key and value per block of P tokens that lies wholly before the window;
    ``talk`` float32 ``[heads, heads]``: the heads' softmax weights are mixed, ``w'_h = sum_g talk[h, g] w_g``
    (``scratch`` float32 ``[T, heads, kv heads, vd]``).  float32 arithmetic; q, caches and out in one dtype.
    A step of few tokens (single tokens of a few requests) cuts every token's keys into ``n_split`` ranges that
    run as warps of their own and are joined by a second launch (None: chosen from the step's size).
    A step with long portions (``n_requests`` given, at least 32 tokens and 8 a request on average) of shapes that
    ``window_attention_uses_tensor_cores`` takes runs scores and sums on the tensor cores; ``tensor_cores`` True
    forces that path (and raises where it cannot run), False keeps the CUDA cores."""
    T, nq, hd = q.shape
    num_pages, nkv, page_size, hd2 = k_cache.shape
    vd = v_cache.shape[3]
    if hd2 != hd or tuple(out.shape) != (T, nq, vd) or out.dtype != q.dtype or k_cache.dtype != q.dtype:
        raise ValueError("window_attention: shape/dtype mismatch")
    n_pool_pages = 0
    if pool_table is not None:
        if pool <= 0 or pooled_k is None or pooled_v is None or tuple(pooled_k.shape[1:]) != (nkv, page_size, hd) \
                or tuple(pooled_v.shape[1:]) != (nkv, page_size, vd) or pooled_k.dtype != q.dtype:
            raise ValueError("window_attention: the pooled pages do not fit")
        _want(pool_table, torch.int32, "pool_table")
        n_pool_pages = pooled_k.shape[0]
    if dist_bias is not None:
        _want(dist_bias, torch.float32, "dist_bias")
        if tuple(dist_bias.shape) != (window, nq):
            raise ValueError("window_attention: dist_bias must be [window, heads]")
    if sink is not None:
        _want(sink, torch.float32, "sink")
        if sink.numel() != nq:
            raise ValueError("window_attention: sink must have one number a head")
    if talk is not None:
        _want(talk, torch.float32, "talk"); _want(scratch, torch.float32, "scratch")
        if tuple(talk.shape) != (nq, nq) or scratch.numel() < T * nq * nkv * vd:
            raise ValueError("window_attention: talk must be [heads, heads] and scratch [T, heads, kv heads, vd]")
    mma = tensor_cores is not False and window_attention_uses_tensor_cores(q.dtype, hd, vd) and (
        tensor_cores or (n_requests is not None and T >= 32 and T >= 8 * n_requests))
    if tensor_cores and not mma:
        raise ValueError("window_attention: these shapes or dtypes do not run on the tensor cores")
    if mma:
        _check(lib().qb_window_attention_mma(
            _p(q), _code(q), _p(k_cache), _p(v_cache), _p(pooled_k), _p(pooled_v), _p(out), _p(scratch), _p(talk),
            _p(tok_pos), _p(tok_req), _p(block_table), block_table.shape[1], _p(pool_table),
            pool_table.shape[1] if pool_table is not None else 0, T, nq, nkv, hd, vd, page_size, num_pages, n_pool_pages,
            ctypes.c_float(scale), ctypes.c_float(softcap), int(window), int(pool), _p(dist_bias), _p(sink), _p(status),
            _stream()), "window_attention_mma", 1 + (talk is not None))
        return
    if n_split is None:
        warps = T * nkv * (nkv if talk is not None else 1)        # of the kernel that shares a key row among q heads
        n_split = 1 if window <= 0 else max(1, min(-(-8192 // warps), -(-window // 32), 64))
    part = None
    if n_split > 1:
        part = torch.empty(T * nq * n_split * (2 + (nkv if talk is not None else 1) * vd), dtype=torch.float32,
                           device=q.device)
    _check(lib().qb_window_attention(
        _p(q), _code(q), _p(k_cache), _p(v_cache), _p(pooled_k), _p(pooled_v), _p(out), _p(scratch), _p(talk),
        _p(tok_pos), _p(tok_req), _p(block_table), block_table.shape[1], _p(pool_table),
        pool_table.shape[1] if pool_table is not None else 0, T, nq, nkv, hd, vd, page_size, num_pages, n_pool_pages,
        ctypes.c_float(scale), ctypes.c_float(softcap), int(window), int(pool), _p(dist_bias), _p(sink), _p(part),
        int(n_split), _p(status), _stream()), "window_attention", 1 + (talk is not None) + (n_split > 1))


def pool_blocks(k_cache, v_cache, pooled_k, pooled_v, tok_pos, tok_req, block_table, pool_table, pool: int, status) -> None:
    """Every token of the step whose position ends a block of ``pool`` tokens leaves the mean key and mean value of
    the block (as the cache holds them) in row ``position // pool`` of the pooled pages."""
    num_pages, nkv, page_size, hd = k_cache.shape
    vd = v_cache.shape[3]
    if tuple(pooled_k.shape[1:]) != (nkv, page_size, hd) or tuple(pooled_v.shape[1:]) != (nkv, page_size, vd) \
            or pooled_k.dtype != k_cache.dtype:
        raise ValueError("pool_blocks: the pooled pages do not fit")
    _check(lib().qb_pool_blocks(_p(k_cache), _p(v_cache), _p(pooled_k), _p(pooled_v), _code(k_cache), _p(tok_pos),
                                _p(tok_req), _p(block_table), block_table.shape[1], _p(pool_table), pool_table.shape[1],
                                tok_pos.numel(), nkv, hd, vd, page_size, num_pages, pooled_k.shape[0], int(pool),
                                _p(status), _stream()), "pool_blocks")


# ---- selective state-space scan (csrc/selective_scan.cu) ----------------------------------------------------------
SCAN_MAX_STATE = 256


def selective_scan(u, proj, z, dt_pre, dt_bias, A, D, state, out, req_start, req_slot, rank: int, n_state: int) -> None:
    """``S <- exp(dt A) S + dt u B``, ``y = S C + D u``, ``out = y * silu(z)`` per channel over each request's rows, with
    ``dt = softplus(dt_pre + dt_bias)``.  ``u`` ``[T, inner]`` in the activation dtype; ``proj`` float32 rows
    ``[low (rank) | B (n_state) | C (n_state)]``; ``z`` float32 ``[T, inner]`` (a column range of wider rows is fine);
    ``dt_pre`` float32 ``[T, inner]``, the step projection of ``low``; ``A`` float32 ``[inner, n_state]`` (negative);
    ``state`` float32 ``[slots, inner, n_state]``, read and left updated at the rows ``req_slot``."""
    T, inner = u.shape
    for t, n in ((proj, "proj"), (z, "z"), (dt_pre, "dt_pre"), (dt_bias, "dt_bias"), (A, "A"), (D, "D"), (state, "state")):
        _want(t, torch.float32, n)
    if (proj.shape[0] != T or proj.shape[1] < rank + 2 * n_state or proj.stride(1) != 1 or tuple(z.shape) != (T, inner)
            or z.stride(1) != 1 or tuple(dt_pre.shape) != (T, inner) or not dt_pre.is_contiguous()
            or tuple(A.shape) != (inner, n_state) or D.numel() != inner or dt_bias.numel() != inner
            or tuple(state.shape[1:]) != (inner, n_state) or tuple(out.shape) != (T, inner) or out.dtype != u.dtype):
        raise ValueError("selective_scan: shape mismatch")
    _check(lib().qb_selective_scan(_p(u), _code(u), ctypes.c_void_p(proj.data_ptr()), int(proj.stride(0)),
                                   ctypes.c_void_p(z.data_ptr()), int(z.stride(0)), _p(dt_pre), _p(dt_bias), _p(A), _p(D),
                                   _p(state), _p(out), _p(req_start), _p(req_slot), T, req_slot.numel(), inner,
                                   int(n_state), int(rank), _stream()), "selective_scan")


# ---- grouped norms with branch norms and the depth-weighted stream; caps and gated activations ------------------
NORM_MAX_GROUPS = 64


def grouped_normed_add(h, *, y=None, y_scale: float = 1.0, y_bias=None, y_gain=None, extra=None, extra_scale: float = 1.0,
                       extra_bias=None, extra_gain=None, branch_eps: float = 0.0, gain=None, groups: int = 1,
                       gain_eps: float = 0.0, history=None, n_history: int = 0, history_weights=None, weight=None,
                       weight_groups: int = 1, eps: float = 0.0, out=None, rows=None, store_h: bool = True) -> None:
    """One launch for what lies between two sublayers (all float32; ``h`` ``[T, H]`` is the residual stream):

    ``a = sum_s y[:, s] + y_bias``, ``b = extra + extra_bias``; each is divided by its root mean square over the row
    (``branch_eps`` inside the root) and multiplied by its gain when ``y_gain`` / ``extra_gain`` is given;
    ``z = y_scale * a + extra_scale * b``; ``d = gain * z / rms_g(z)`` where the row is cut into ``groups`` equal
    parts that are each divided by their own root mean square (``gain`` None: ``d = z``); ``x = h + d``.  With
    ``history`` (float32 ``[entries, T, H]``): entry ``n_history`` receives ``x`` and ``x`` becomes
    ``sum_{j <= n_history} history_weights[j] * history[j]``.  ``h`` is stored unless ``store_h`` is False;
    ``out`` (any activation dtype) receives ``weight * x / rms_g(x)`` (``weight_groups`` parts), or ``x`` itself when
    ``weight`` is None.  ``rows`` (int32) selects token rows for ``out`` (not with ``history``)."""
    _want(h, torch.float32, "h")
    T, H = h.shape
    S = 1
    if y is not None:
        _want(y, torch.float32, "y")
        S = y.shape[1] if y.dim() == 3 else 1
        if y.shape[0] != T or y.shape[-1] != H:
            raise ValueError("grouped_normed_add: y shape mismatch")
    elif extra is not None or gain is not None:
        raise ValueError("grouped_normed_add: a second addend or a gain without a first addend")
    for t, n, size in ((y_bias, "y_bias", H), (y_gain, "y_gain", H), (extra, "extra", T * H), (extra_bias, "extra_bias", H),
                       (extra_gain, "extra_gain", H), (gain, "gain", H), (weight, "weight", H)):
        if t is not None:
            _want(t, torch.float32, n)
            if t.numel() != size:
                raise ValueError(f"grouped_normed_add: {n} holds {t.numel()} numbers, {size} wanted")
    for g in (groups, weight_groups):
        if not 1 <= int(g) <= NORM_MAX_GROUPS or H % int(g):
            raise ValueError(f"grouped_normed_add: {g} groups do not divide a width of {H} (1 to {NORM_MAX_GROUPS})")
    hist_stride = 0
    if history is not None:
        _want(history, torch.float32, "history"); _want(history_weights, torch.float32, "history_weights")
        if history.dim() != 3 or tuple(history.shape[1:]) != (T, H) or not 0 <= n_history < history.shape[0] \
                or history_weights.numel() != n_history + 1 or rows is not None:
            raise ValueError("grouped_normed_add: history shape mismatch")
        hist_stride = T * H
    n = T if rows is None else rows.numel()
    if rows is not None:
        _want(rows, torch.int32, "rows")
    if out is not None and (out.shape[0] != n or out.shape[1] != H):
        raise ValueError("grouped_normed_add: out shape mismatch")
    _check(lib().qb_grouped_normed_add(
        _p(h), _p(y), S, ctypes.c_float(y_scale), _p(y_bias), _p(y_gain), _p(extra), ctypes.c_float(extra_scale),
        _p(extra_bias), _p(extra_gain), ctypes.c_float(branch_eps), _p(gain), int(groups), ctypes.c_float(gain_eps),
        _p(history), ctypes.c_longlong(hist_stride), int(n_history), _p(history_weights),
        _p(weight) if out is not None else ctypes.c_void_p(0), int(weight_groups), ctypes.c_float(eps), _p(out),
        _code(out) if out is not None else F32, _p(rows), n, H, int(store_h), _stream()), "grouped_normed_add")


def tanh_cap(x: torch.Tensor, cap: float) -> None:
    """``x <- cap * tanh(x / cap)`` in place (float32)."""
    _want(x, torch.float32, "x")
    _check(lib().qb_tanh_cap(_p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()), "tanh_cap")


GLU_SILU, GLU_CLAMPED = 0, 1


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, *, bias=None, kind: int = GLU_SILU, limit: float = 0.0,
            alpha: float = 1.0) -> None:
    """The activation of a gated dense feed-forward from ``gate_up`` ``[n, 2 I]`` = ``[gate | up]`` (the activation
    dtype, or the product's float32 accumulators) into ``out`` ``[n, I]``; ``bias`` float32 ``[2 I]`` is added first.
    ``GLU_SILU``: ``silu(gate) * up``; ``GLU_CLAMPED``: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``,
    ``g * sigmoid(alpha * g) * (u + 1)``."""
    n, two_i = gate_up.shape
    if tuple(out.shape) != (n, two_i // 2) or (gate_up.dtype != out.dtype and gate_up.dtype != torch.float32):
        raise ValueError("glu_act: shape/dtype mismatch")
    if bias is not None:
        _want(bias, torch.float32, "bias")
        if bias.numel() != two_i:
            raise ValueError("glu_act: the bias has 2 I numbers")
    if kind == GLU_CLAMPED and not limit > 0:
        raise ValueError("glu_act: the clamped form needs a positive limit")
    _check(lib().qb_glu_act(_p(gate_up), _code(gate_up), _p(bias), _p(out), _code(out), n, two_i // 2, int(kind),
                            ctypes.c_float(limit), ctypes.c_float(alpha), _stream()), "glu_act")


GATED_DELTA_MAX_DIM = 256


def gated_delta(qkv, ab, a_off: int, b_off: int, A_log, dt_bias, state, out, req_start, req_slot, n_heads: int,
                n_groups: int, dim: int, vdim: int, q_scale: float, unit_eps: float) -> None:
    """The recurrence ``S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` per (request, head) over the
    step's tokens, from and into ``state`` ``[slots, heads, dim, vdim]`` float32.  ``qkv`` float32 ``[T, P]`` holds
    ``q | k`` (groups x dim each; head h reads group ``h // (heads / groups)``) and ``v`` (heads x vdim) in its
    first columns, after convolution and activation; q and k are made unit vectors per group here (``unit_eps``
    under the root), q also times ``q_scale``.  ``ab`` float32 rows whose columns ``a_off + h`` / ``b_off + h`` are
    the pre-activations of the decay ``g = exp(-exp(A_log) * softplus(a + dt_bias))`` and of ``beta = sigmoid(b)``.
    ``out`` float32 ``[T, heads, vdim]``."""
    for t, n in ((qkv, "qkv"), (ab, "ab"), (A_log, "A_log"), (dt_bias, "dt_bias"), (state, "state"), (out, "out")):
        _want(t, torch.float32, n)
    T = qkv.shape[0]
    H, G, D, DV = int(n_heads), int(n_groups), int(dim), int(vdim)
    if (qkv.stride(1) != 1 or ab.stride(1) != 1 or qkv.shape[1] < 2 * G * D + H * DV or ab.shape[0] != T
            or min(a_off, b_off) < 0 or max(a_off, b_off) + H > ab.shape[1] or out.numel() != T * H * DV
            or A_log.numel() != H or dt_bias.numel() != H or tuple(state.shape[1:]) != (H, D, DV) or H % G):
        raise ValueError("gated_delta: shape mismatch")
    R = req_slot.numel()
    scratch = torch.empty(T * (2 * G * D + 2 * H), dtype=torch.float32, device=qkv.device)
    _check(lib().qb_gated_delta(ctypes.c_void_p(qkv.data_ptr()), int(qkv.stride(0)), ctypes.c_void_p(ab.data_ptr()),
                                int(ab.stride(0)), int(a_off), int(b_off), _p(A_log), _p(dt_bias), _p(state), _p(out),
                                _p(scratch), _p(req_start), _p(req_slot), R, T, H, G, D, DV, ctypes.c_float(q_scale),
                                ctypes.c_float(unit_eps), _stream()), "gated_delta", 2)
