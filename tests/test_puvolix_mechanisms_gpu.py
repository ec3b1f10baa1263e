"""Every mechanism of the Puvolix decoder alone: the framework's kernel or part against the plain function of the
same mechanism (tests/plain/puvolix_plain.py), for prompts, portions and single tokens, on caches whose pages are
shuffled and state slots that were used before.  Where random numbers would hide a fault the inputs are made so that
it shows: one key whose score outweighs all others sits at position 0, at a page's first and last place, and far
back among hundreds."""

import math

import pytest
import torch

from tests.plain import puvolix_plain as P

DEV = "cuda:0"
gpu = pytest.mark.gpu


def _close(got, want, tol, what=""):
    scale = float(want.abs().max()) or 1.0
    err = float((got.float().cpu() - want.float().cpu()).abs().max()) / scale
    assert err < tol, (what, err)


# ---- norms in groups, branch norms, the depth-weighted stream ---------------------------------------------------
@gpu
@pytest.mark.parametrize("H,groups,out_groups", [(48, 3, 1), (256, 4, 4), (40, 1, 5), (1536, 6, 2), (66, 2, 3)])
def test_grouped_norm_between_sublayers(H, groups, out_groups):
    from quanta_b200 import kernels
    g = torch.Generator().manual_seed(H)
    T, S = 7, 3
    rnd = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    h, y, extra = rnd(T, H), rnd(T, S, H) * 3, rnd(T, H) * 0.2
    y_bias, e_bias, y_gain, e_gain, gain, weight = rnd(H), rnd(H), rnd(H), rnd(H), rnd(H), rnd(H)
    eps_b, eps_y, eps = 1e-3, 1e-2, 1e-5
    a = P.rms(y.sum(1) + y_bias, eps_b) * y_gain
    b = P.rms(extra + e_bias, eps_b) * e_gain
    z = 0.5 * a + 0.25 * b
    x = h + P.grouped_norm(z, gain, groups, eps_y)
    want_out = P.grouped_norm(x, weight, out_groups, eps)
    d = lambda t: t.to(DEV)  # noqa: E731
    hd = d(h.clone())
    for dtype in (torch.float32, torch.bfloat16):
        hd = d(h.clone())
        out = torch.empty((T, H), dtype=dtype, device=DEV)
        kernels.grouped_normed_add(hd, y=d(y), y_scale=0.5, y_bias=d(y_bias), y_gain=d(y_gain), extra=d(extra),
                                   extra_scale=0.25, extra_bias=d(e_bias), extra_gain=d(e_gain), branch_eps=eps_b,
                                   gain=d(gain), groups=groups, gain_eps=eps_y, weight=d(weight), weight_groups=out_groups,
                                   eps=eps, out=out)
        _close(hd, x, 2e-6, "stream")
        _close(out, want_out, 2e-6 if dtype == torch.float32 else 1e-2, "normed")
    # wanted rows only, the stream left as it was; no norm of the output: the stream itself comes out
    rows = torch.tensor([5, 0, 3], dtype=torch.int32, device=DEV)
    hd = d(h.clone())
    out = torch.empty((3, H), dtype=torch.float32, device=DEV)
    kernels.grouped_normed_add(hd, y=d(y), gain=d(gain), groups=groups, gain_eps=eps_y, weight=d(weight),
                               weight_groups=out_groups, eps=eps, out=out, rows=rows, store_h=False)
    x2 = h + P.grouped_norm(y.sum(1), gain, groups, eps_y)
    _close(out, P.grouped_norm(x2, weight, out_groups, eps)[[5, 0, 3]], 2e-6, "rows")
    _close(hd, h, 1e-9, "stream untouched")
    out = torch.empty((T, H), dtype=torch.float32, device=DEV)
    kernels.grouped_normed_add(hd, out=out)
    _close(out, h, 1e-9, "the stream itself")


@gpu
def test_depth_weighted_stream():
    """Three layers' results and the embedding output: after each layer the stream is the weighted sum so far."""
    from quanta_b200 import kernels
    g = torch.Generator().manual_seed(5)
    T, H, L = 5, 72, 3
    x0 = torch.randn(T, H, generator=g)
    hist = torch.full((L + 1, T, H), 99.0, device=DEV)        # stale numbers
    hist[0] = x0.to(DEV)
    h = x0.clone().to(DEV)
    results, x = [x0], x0
    for i in range(L):
        y = torch.randn(T, H, generator=g)
        gain = torch.randn(H, generator=g)
        w = torch.randn(i + 2, generator=g)
        res = x + P.grouped_norm(y, gain, 4, 1e-5)
        results.append(res)
        x = sum(w[j] * results[j] for j in range(i + 2))
        kernels.grouped_normed_add(h, y=y.to(DEV), gain=gain.to(DEV), groups=4, gain_eps=1e-5, history=hist,
                                   n_history=i + 1, history_weights=w.to(DEV))
        _close(h, x, 3e-6, f"layer {i}")
        _close(hist[i + 1], res, 3e-6, f"result {i}")


@gpu
def test_capped_logits_and_gated_activations():
    from quanta_b200 import kernels
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 50, generator=g) * 40
    xd = x.clone().to(DEV)
    kernels.tanh_cap(xd, 30.0)
    _close(xd, 30.0 * torch.tanh(x / 30.0), 1e-6)
    gu, bias = torch.randn(6, 2 * 20, generator=g) * 2, torch.randn(40, generator=g)
    a, b = gu[:, :20] + bias[:20], gu[:, 20:] + bias[20:]
    out = torch.empty((6, 20), device=DEV)
    kernels.glu_act(gu.to(DEV), out, bias=bias.to(DEV))
    _close(out, torch.nn.functional.silu(a) * b, 1e-6, "silu with biases")
    a, b = torch.clamp(gu[:, :20], max=0.9), torch.clamp(gu[:, 20:], -0.9, 0.9)
    kernels.glu_act(gu.to(DEV), out, kind=kernels.GLU_CLAMPED, limit=0.9, alpha=1.702)
    _close(out, a * torch.sigmoid(1.702 * a) * (b + 1), 1e-6, "clamped")


# ---- short convolutions and their state ---------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("taps,silu", [(1, False), (2, True), (3, False), (4, True), (6, False)])
def test_short_convolution_across_portions(taps, silu):
    """Two sequences in portions down to one token, in slots that hold another sequence's inputs: every row equals
    the convolution of the whole sequence."""
    from quanta_b200 import kernels
    g = torch.Generator().manual_seed(taps)
    C, lens = 21, [23, 9]
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, C + 3, generator=g) for n in lens]           # rows wider than the channels that count
    want = [P.causal_conv(s[:, :C], w) for s in seqs]
    if silu:
        want = [torch.nn.functional.silu(t) for t in want]
    state = torch.full((3, taps - 1, C), 50.0, device=DEV)
    slots = [2, 0]
    for s in slots:
        state[s].zero_()                                                # what admission does
    done = [0, 0]
    cuts = [[1, 2, 1, 7, 2, 10], [2, 1, 1, 5]]
    got = [[], []]
    for step in range(6):
        rows, req, start, slot, who = [], [], [0], [], []
        for r in (0, 1):
            if step < len(cuts[r]):
                n = cuts[r][step]
                rows.append(seqs[r][done[r]: done[r] + n])
                req += [len(who)] * n
                start.append(start[-1] + n)
                slot.append(slots[r])
                who.append((r, n))
                done[r] += n
        x = torch.cat(rows).to(DEV)
        out = torch.empty((x.shape[0], C), device=DEV)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
        kernels.short_conv(x[:, :C], w.to(DEV), state, out, i32(req), i32(start), i32(slot), silu=silu, plain=not silu)
        at = 0
        for r, n in who:
            got[r].append(out[at: at + n].cpu())
            at += n
    for r in (0, 1):
        _close(torch.cat(got[r]), want[r], 2e-6, f"sequence {r}")
    assert taps == 1 or float(state[1].min()) == 50.0                   # a slot nobody holds is not touched


def test_rescaled_frequencies():
    """The ladder after rescaling by wavelength, in all three ranges, against the plain function."""
    from quanta_b200.parts.rotary import PartialRotary
    for dims, base, sc in [(40, 130000.0, (6.0, 1.0, 4.0, 1024)), (16, 100.0, (8.0, 0.5, 2.0, 64)), (8, 900.0, (3.0, 1.0, 3.0, 40)),
                           (32, 1e4, None)]:
        part = PartialRotary(head_dim=dims + 8, rotary_dim=dims, theta=base, wavelength_scaling=sc)
        scaling = None if sc is None else dict(zip(("factor", "low", "high", "original"), sc))
        want = P.scaled_frequencies(dims, base, scaling, torch.float64)
        got = part.inv_freq()
        assert got.dtype == torch.float32 and torch.allclose(got.double(), want, rtol=2e-7, atol=0)
        if sc is not None:
            plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
            ratio = (plain / want)
            assert float(ratio.min()) < 1.0 + 1e-9 and float(ratio.max()) > sc[0] - 1e-6     # kept ones and slowed ones
    with pytest.raises(ValueError):
        PartialRotary(head_dim=8, rotary_dim=8, theta=10.0, wavelength_scaling=(2.0, 4.0, 1.0, 64))


# ---- q/k norm, rotation, head temperature, cache write, attention ------------------------------------------------
class Paged:
    """Empty pages in a shuffled order for some sequences; stale numbers everywhere."""

    def __init__(self, lengths, G, hd, vd, page, dtype, seed=0):
        from quanta_b200 import kernels
        per = [-(-n // page) for n in lengths]
        total = sum(per) + 3
        order = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
        self.page = page
        self.k = torch.full((total, G, page, hd), 7.0, dtype=dtype, device=DEV)
        self.v = torch.full((total, G, page, vd), -5.0, dtype=dtype, device=DEV)
        table = torch.full((len(lengths), max(per)), -1, dtype=torch.int32)
        for r in range(len(lengths)):
            for p in range(per[r]):
                table[r, p] = order.pop()
        self.table = table.to(DEV)
        self.status = kernels.new_status(DEV)


def _write(cache, rows, qkv, nq, G, hd, vd, qw, kw, eps, freqs, dims, temp, dtype):
    """The framework's norm + rotation + temperature + cache write for the rows ``(request, position)``."""
    from quanta_b200 import kernels
    T = qkv.shape[0]
    q = torch.empty((T, nq, hd), dtype=dtype, device=DEV)
    req = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    kernels.qknorm_rope_write(qkv.to(DEV), q, cache.k, cache.v, qw.to(DEV), kw.to(DEV), kernels.NORM_PER_HEAD, eps,
                              freqs.to(DEV), None, pos.view(T, 1), pos, req, cache.table, nq, G, hd, dims, cache.page,
                              cache.status, vd=vd, head_scale=None if temp is None else temp.to(DEV))
    assert int(cache.status[0]) == 0
    return q, pos, req


def _attend(cache, q, pos, req, scale, dtype, **opts):
    from quanta_b200 import kernels
    out = torch.empty((q.shape[0], q.shape[1], cache.v.shape[3]), dtype=dtype, device=DEV)
    kernels.window_attention(q, cache.k, cache.v, out, pos, req, cache.table, scale, 0, cache.status, **opts)
    assert int(cache.status[0]) == 0
    return out.float().cpu()


@gpu
@pytest.mark.parametrize("nq,G,hd,vd,dims,page,dtype", [
    (4, 2, 12, 20, 8, 4, torch.float32), (8, 2, 48, 32, 32, 16, torch.bfloat16), (6, 3, 16, 16, 0, 8, torch.float32),
    (2, 2, 64, 64, 32, 16, torch.bfloat16), (3, 1, 10, 6, 10, 5, torch.float32), (4, 1, 96, 64, 64, 16, torch.bfloat16),
    (2, 1, 128, 128, 128, 8, torch.bfloat16), (4, 2, 80, 16, 16, 16, torch.bfloat16), (4, 4, 32, 128, 0, 16, torch.bfloat16),
    (2, 1, 256, 128, 64, 16, torch.bfloat16), (4, 2, 24, 40, 24, 16, torch.bfloat16), (2, 1, 144, 144, 48, 16, torch.bfloat16),
    (6, 2, 32, 32, 16, 16, torch.bfloat16), (5, 1, 64, 32, 64, 8, torch.bfloat16), (12, 4, 16, 48, 8, 16, torch.bfloat16),
    (7, 7, 48, 16, 48, 16, torch.bfloat16), (20, 1, 32, 32, 32, 16, torch.bfloat16)])
def test_attention_of_prompts_portions_and_single_tokens(nq, G, hd, vd, dims, page, dtype):
    """Two sequences: the first as one prompt, the second as a portion and then token by token, through shuffled
    pages; per-head norm gains, rotated part, head temperatures and scale as the plain functions have them."""
    g = torch.Generator().manual_seed(nq * hd)
    lens, eps, scale = [70, 41], 1e-5, 0.37
    qw, kw, temp = torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5, torch.rand(nq, generator=g) + 0.5
    freqs = P.scaled_frequencies(dims, 50.0, None, torch.float32) if dims else torch.empty(0)
    cache = Paged(lens, G, hd, vd, page, dtype, seed=3)
    want, raw = [], []
    for n in lens:
        qkv = torch.randn(n, nq * hd + G * hd + G * vd, generator=g)
        raw.append(qkv)
        pos = torch.arange(n)
        q = P.rms(qkv[:, : nq * hd].view(n, nq, hd), eps) * qw
        k = P.rms(qkv[:, nq * hd: (nq + G) * hd].view(n, G, hd), eps) * kw
        v = qkv[:, (nq + G) * hd:].view(n, G, vd)
        if dims:
            q, k = P.rotate(q, pos, dims, freqs), P.rotate(k, pos, dims, freqs)
        want.append(P.attend(q, k, v, scale, temp))
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    # the first sequence whole, beside a portion of the second: one step, 70 + 30 tokens
    rows = [(0, p) for p in range(70)] + [(1, p) for p in range(30)]
    q, pos, req = _write(cache, rows, torch.cat([raw[0], raw[1][:30]]), nq, G, hd, vd, qw, kw, eps, freqs, dims, temp, dtype)
    out = _attend(cache, q, pos, req, scale, dtype, n_requests=2)
    _close(out[:70], want[0], tol, "prompt")
    _close(out[70:], want[1][:30], tol, "portion")
    # two tokens, then one by one, with the ranges of keys cut in different numbers
    for p0, n, split in [(30, 2, 1), (32, 1, 3), (33, 1, 1), (34, 1, 64), (35, 6, 2)]:
        rows = [(1, p) for p in range(p0, p0 + n)]
        q, pos, req = _write(cache, rows, raw[1][p0: p0 + n], nq, G, hd, vd, qw, kw, eps, freqs, dims, temp, dtype)
        out = _attend(cache, q, pos, req, scale, dtype, n_split=split)
        _close(out, want[1][p0: p0 + n], tol, f"tokens from {p0}")


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("where", [0, 1, 15, 16, 17, 255, 256, 400, 688])
def test_a_key_that_stands_out(where, dtype):
    """Among 700 keys one has a score far above the rest: the query at the end (as the last row of a prompt, and as
    a single token whose keys are cut into ranges) returns that key's value, wherever it lies: the first positions,
    a page's last and first place, far back."""
    g = torch.Generator().manual_seed(where)
    n, nq, G, hd, vd, page = 700, 4, 2, 32, 16, 16
    k = torch.randn(n, G, hd, generator=g) * 0.1
    v = torch.randn(n, G, vd, generator=g)
    q = torch.randn(n, nq, hd, generator=g) * 0.1
    k[where] = 0.0
    k[where, :, 3] = 6.0
    q[-1] = 0.0
    q[-1, :, 3] = 6.0                               # score 36 at ``where`` against about 0 elsewhere
    want = P.attend(q, k, v, 1.0, torch.ones(nq))
    assert float((want[-1] - v[where].repeat_interleave(nq // G, 0)).abs().max()) < 1e-3
    cache = Paged([n], G, hd, vd, page, dtype, seed=where)
    rows = [(0, p) for p in range(n)]
    qkv = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1)
    none = torch.empty(0)
    from quanta_b200 import kernels
    qd = torch.empty((n, nq, hd), dtype=dtype, device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    req = torch.zeros(n, dtype=torch.int32, device=DEV)
    kernels.qknorm_rope_write(qkv.to(DEV), qd, cache.k, cache.v, None, None, kernels.NORM_NONE, 0.0, none.to(DEV), None,
                              pos.view(n, 1), pos, req, cache.table, nq, G, hd, 0, page, cache.status, vd=vd)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    out = _attend(cache, qd, pos, req, 1.0, dtype, n_requests=1)
    _close(out[-1], want[-1], tol, "last row of the prompt")
    _close(out[where], want[where], tol, "the key's own row")
    for split in (1, 5, 22):
        one = _attend(cache, qd[-1:].contiguous(), pos[-1:].contiguous(), req[-1:].contiguous(), 1.0, dtype, n_split=split)
        _close(one[0], want[-1], tol, f"single token, {split} ranges")


# ---- the gated delta rule -------------------------------------------------------------------------------------
@gpu
@pytest.mark.parametrize("H,G,D,DV", [(4, 2, 12, 20), (4, 4, 64, 32), (2, 1, 24, 8), (3, 3, 10, 14), (8, 2, 128, 64), (1, 1, 40, 130)])
def test_gated_delta_rule_in_portions(H, G, D, DV):
    """Two sequences in unequal portions and single tokens, in slots that hold stale states, against the plain
    recurrence over the whole sequences; the state that is left equals the plain one."""
    from quanta_b200 import kernels
    g = torch.Generator().manual_seed(H * D + DV)
    lens = [37, 12]
    C = 2 * G * D + H * DV
    A_log, dt_bias = torch.rand(H, generator=g) * 2 - 1.5, torch.randn(H, generator=g)
    seqs, want, want_S = [], [], []
    for n in lens:
        qkv = torch.randn(n, C + 5, generator=g)
        ab = torch.randn(n, 2 * H + 3, generator=g) * 2                  # [.. a (H) | b (H) ..] from column 1
        seqs.append((qkv, ab))
        q, k = qkv[:, : G * D].view(n, G, D), qkv[:, G * D: 2 * G * D].view(n, G, D)
        v = qkv[:, 2 * G * D: C].view(n, H, DV)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        decay = torch.exp(-torch.exp(A_log) * torch.nn.functional.softplus(ab[:, 1: 1 + H] + dt_bias))
        beta = torch.sigmoid(ab[:, 1 + H: 1 + 2 * H])
        o, S = P.delta_recurrence(q.double(), k.double(), v.double(), decay.double(), beta.double())
        want.append(o.float())
        want_S.append(S.float())
    state = torch.full((3, H, D, DV), 3.0, device=DEV)
    slots = [1, 2]
    for s in slots:
        state[s].zero_()
    cuts = [[5, 1, 1, 2, 17, 1, 10], [1, 2, 9]]
    done, got = [0, 0], [[], []]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    for step in range(7):
        rows_q, rows_ab, start, slot, who = [], [], [0], [], []
        for r in (0, 1):
            if step < len(cuts[r]):
                n = cuts[r][step]
                rows_q.append(seqs[r][0][done[r]: done[r] + n])
                rows_ab.append(seqs[r][1][done[r]: done[r] + n])
                start.append(start[-1] + n)
                slot.append(slots[r])
                who.append((r, n))
                done[r] += n
        qkv, ab = torch.cat(rows_q).to(DEV), torch.cat(rows_ab).to(DEV)
        out = torch.empty((qkv.shape[0], H, DV), device=DEV)
        kernels.gated_delta(qkv, ab, 1, 1 + H, A_log.to(DEV), dt_bias.to(DEV), state, out, i32(start), i32(slot), H, G, D, DV,
                            D ** -0.5, 1e-6)
        at = 0
        for r, n in who:
            got[r].append(out[at: at + n].cpu())
            at += n
    for r in (0, 1):
        _close(torch.cat(got[r]), want[r], 2e-5, f"sequence {r}")
        _close(state[slots[r]], want_S[r], 2e-5, f"state {r}")
    assert float(state[0].min()) == 3.0


# ---- routed experts whose weight multiplies the input ------------------------------------------------------------
class _Ctx:
    def __init__(self):
        from quanta_b200 import kernels
        self.status = kernels.new_status(DEV)


@gpu
@pytest.mark.parametrize("T,W,E,top,ff,shared,dtype", [(9, 40, 5, 2, 24, (16, 0.8), torch.float32), (150, 64, 8, 1, 64, (128, 1.0), torch.bfloat16),
                                                   (5, 48, 5, 2, 24, (16, 0.8), torch.bfloat16), (1, 64, 4, 3, 16, None, torch.bfloat16),
                                                   (3, 24, 3, 3, 8, None, torch.float32), (40, 128, 6, 2, 32, None, torch.bfloat16)])
def test_input_weighted_experts(T, W, E, top, ff, shared, dtype):
    """The part alone: choice, scores, the weight on the expert's input, both clamps, the shared expert."""
    from quanta_b200.parts.base import make
    from quanta_b200 import matmul
    matmul.configure()
    g = torch.Generator().manual_seed(T + W)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 0.7},
           "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}
    w = {"router": torch.randn(E, W, generator=g) * 3 / math.sqrt(W)}
    for e in range(E):
        w.update({f"e{e}.gate": torch.randn(ff, W, generator=g) * 2 / math.sqrt(W), f"e{e}.up": torch.randn(ff, W, generator=g) * 2 / math.sqrt(W),
                  f"e{e}.down": torch.randn(W, ff, generator=g) / math.sqrt(ff)})
    if shared is not None:
        w.update({"shared.gate": torch.randn(shared[0], W, generator=g) * 2 / math.sqrt(W),
                  "shared.up": torch.randn(shared[0], W, generator=g) * 2 / math.sqrt(W),
                  "shared.down": torch.randn(W, shared[0], generator=g) / math.sqrt(shared[0])})
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    part = make("feed_forward", ("input_weighted_experts", dict(
        hidden_size=W, expert_size=ff, n_experts=E, top_k=top, limit=0.7, alpha=1.702,
        shared_size=0 if shared is None else shared[0], shared_limit=0.0 if shared is None else shared[1],
        names={"gate": "router", "w1": "e{e}.gate", "w3": "e{e}.up", "w2": "e{e}.down", "shared_gate": "shared.gate",
               "shared_up": "shared.up", "shared_down": "shared.down"})))
    kinds = {s.name: s.kind for p in [part, *part.children()] for s in p.tensor_specs()}
    fetch = lambda n: w[n].to(DEV, torch.float32 if kinds[n] == "f32" else dtype)  # noqa: E731
    part.load(fetch)
    for child in part.children():
        child.load(fetch)
    x = (torch.randn(T, W, generator=g)).to(dtype)
    part.trace = []
    got = part.forward(x.to(DEV), _Ctx()).total().cpu()
    chosen = part.trace[0].cpu()
    want, idx, margin = P.routed_ff(w, "", x.float(), mlp, chosen=chosen)
    clear = margin > (1e-5 if dtype == torch.float32 else 2e-2)
    _, own, _ = P.routed_ff(w, "", x.float(), mlp)
    assert bool((own[clear] == chosen[clear].long()).all())             # the engine chose what the plain router chooses
    _close(got, want, 3e-5 if dtype == torch.float32 else 3e-2)
