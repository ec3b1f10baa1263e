"""Every mechanism of the Tarulix decoder alone: the framework's kernel against the plain function of the same
mechanism (tests/plain/tarulix_plain.py), on caches whose pages are shuffled, for prompts, portions and single
tokens.  Where random numbers would hide a fault the inputs are made so that it shows: one key whose score
outweighs all others sits just inside and just outside a window, at a page border, far back, in a pooled block
that is just seen or not yet, or among the tokens that no longer count at all.
"""

import math

import pytest
import torch

from tests.plain import tarulix_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


# ---- a paged cache filled from whole sequences -------------------------------------------------------------
class Paged:
    """Keys and values of some sequences laid into shuffled pages (and the pooled rows of their whole blocks)."""

    def __init__(self, ks, vs, page, dtype, pool=0, seed=0):
        from quanta_b200 import kernels
        self.page, self.pool, self.dtype = page, pool, dtype
        G, hd, vd = ks[0].shape[1], ks[0].shape[2], vs[0].shape[2]
        per = [-(-k.shape[0] // page) for k in ks]
        total = sum(per) + 3
        g = torch.Generator().manual_seed(seed)
        order = torch.randperm(total, generator=g).tolist()
        self.k = torch.full((total, G, page, hd), 7.0, dtype=dtype, device=DEV)       # stale numbers everywhere
        self.v = torch.full((total, G, page, vd), -5.0, dtype=dtype, device=DEV)
        self.table = torch.full((len(ks), max(per)), -1, dtype=torch.int32)
        for r, (k, v) in enumerate(zip(ks, vs)):
            for p in range(per[r]):
                pg = order.pop()
                self.table[r, p] = pg
                n = min(page, k.shape[0] - p * page)
                self.k[pg, :, :n] = k[p * page: p * page + n].transpose(0, 1).to(dtype).to(DEV)
                self.v[pg, :, :n] = v[p * page: p * page + n].transpose(0, 1).to(dtype).to(DEV)
        self.table = self.table.to(DEV)
        self.status = kernels.new_status(DEV)
        self.kp = self.vp = self.ptable = None
        if pool:
            pper = [max(1, -(-(k.shape[0] // pool) // page)) for k in ks]
            ptotal = sum(pper) + 2
            porder = torch.randperm(ptotal, generator=g).tolist()
            self.kp = torch.full((ptotal, G, page, hd), 3.0, dtype=dtype, device=DEV)
            self.vp = torch.full((ptotal, G, page, vd), 9.0, dtype=dtype, device=DEV)
            self.ptable = torch.full((len(ks), max(pper)), -1, dtype=torch.int32)
            for r in range(len(ks)):
                for p in range(pper[r]):
                    self.ptable[r, p] = porder.pop()
            self.ptable = self.ptable.to(DEV)

    def fill_pooled(self, lengths):
        """Run the framework's block-mean kernel for every position of every sequence."""
        from quanta_b200 import kernels
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lengths]).to(DEV)
        req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(lengths)]).to(DEV)
        kernels.pool_blocks(self.k, self.v, self.kp, self.vp, pos, req, self.table, self.ptable, self.pool, self.status)


def _rounded(t, dtype):
    return t.to(dtype).float()


def _attend(cache, q, rows, scale, window, dtype, **opts):
    """``rows``: (request, position) of every query row of ``q`` [T, H, hd]."""
    from quanta_b200 import kernels
    T, Hq, _ = q.shape
    G, vd = cache.v.shape[1], cache.v.shape[3]
    out = torch.empty((T, Hq, vd), dtype=dtype, device=DEV)
    req = torch.tensor([r for r, _ in rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device=DEV)
    if opts.get("talk") is not None:
        opts["scratch"] = torch.empty((T, Hq, G, vd), dtype=torch.float32, device=DEV)
    if cache.pool:
        opts.update(pool=cache.pool, pooled_k=cache.kp, pooled_v=cache.vp, pool_table=cache.ptable)
    kernels.window_attention(q.to(dtype).to(DEV), cache.k, cache.v, out, pos, req, cache.table, scale, window,
                             cache.status, n_split=1, tensor_cores=False, **opts)
    # the other ways the same launch can run: the keys of every token cut into ranges that are joined afterwards
    # (steps of few tokens), and scores and sums on the tensor cores (long portions, the shapes that path takes);
    # each must give what one warp a (token, head) gives
    others = {"ranges_2": dict(n_split=2, tensor_cores=False), "ranges_7": dict(n_split=7, tensor_cores=False)}
    if kernels.window_attention_uses_tensor_cores(dtype, q.shape[2], vd):
        others["tensor_cores"] = dict(tensor_cores=True)
    tol = 2e-5 if dtype == torch.float32 else 1.6e-2
    for name, how in others.items():
        alt = torch.full_like(out, float("nan"))
        kernels.window_attention(q.to(dtype).to(DEV), cache.k, cache.v, alt, pos, req, cache.table, scale, window,
                                 cache.status, **how, **opts)
        assert torch.allclose(alt.float(), out.float(), atol=tol, rtol=tol), (name, float((alt.float() - out.float()).abs().max()))
    torch.cuda.synchronize()
    assert int(cache.status.cpu()[0]) == 0
    return out.float().cpu()


def _bias_rows_by_distance(rel, window, far):
    """The table as the kernel takes it: one row per distance below the window."""
    return torch.stack([rel[P.distance_bucket(n, rel.shape[0], far)] for n in range(window)]).contiguous()


SHAPES = [
    # heads, kv heads, key size, value size, window, page
    (4, 2, 16, 24, 9, 4), (6, 1, 20, 12, 33, 8), (3, 3, 64, 64, 17, 16), (8, 2, 128, 64, 70, 16), (2, 1, 40, 8, 1, 4),
    (4, 4, 64, 128, 200, 16), (4, 2, 48, 80, 40, 8), (2, 1, 96, 96, 72, 16), (4, 1, 256, 112, 100, 16), (2, 2, 16, 16, 64, 4),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,G,hd,vd,window,page", SHAPES)
def test_distance_bias_and_sink(Hq, G, hd, vd, window, page, dtype):
    """Windowed softmax with the learned bias by bucketed distance and the sink: prompts of three lengths in one
    launch, every position a query."""
    g = torch.Generator().manual_seed(hd + window)
    lengths = [5, 77, 130]
    rows_b, far = 10, max(12.0, 1.5 * window)
    rel = torch.randn(rows_b, Hq, generator=g)
    sink = 0.5 + torch.randn(Hq, generator=g)
    qs = [_rounded(torch.randn(n, Hq, hd, generator=g), dtype) for n in lengths]
    ks = [_rounded(torch.randn(n, G, hd, generator=g), dtype) for n in lengths]
    vs = [_rounded(torch.randn(n, G, vd, generator=g), dtype) for n in lengths]
    scale = 1.3 / math.sqrt(hd)
    cache = Paged(ks, vs, page, dtype, seed=1)
    rows = [(r, p) for r, n in enumerate(lengths) for p in range(n)]
    got = _attend(cache, torch.cat(qs), rows, scale, window, dtype, dist_bias=_bias_rows_by_distance(rel, window, far).to(DEV),
                  sink=sink.to(DEV))
    want = torch.cat([P.biased_sink_rows(q, k, v, window, scale, rel, far, sink) for q, k, v in zip(qs, ks, vs)])
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())
    # without the sink and without the bias the result differs: neither is left out silently
    plain = _attend(cache, torch.cat(qs), rows, scale, window, dtype)
    assert float((plain - want).abs().max()) > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,G,hd,vd,window,page", SHAPES)
@pytest.mark.parametrize("pool,cap,mix", [(3, 0.0, False), (4, 2.0, True), (1, 0.7, True), (16, 0.0, True)])
def test_pooled_blocks_cap_and_mixed_heads(Hq, G, hd, vd, window, page, dtype, pool, cap, mix):
    """Window and pooled blocks in one softmax, the tanh cap, and the heads' weights mixed by a matrix."""
    g = torch.Generator().manual_seed(hd + window + pool)
    lengths = [2, 61, 150]
    talk = (0.6 * torch.eye(Hq) + 0.4 * torch.randn(Hq, Hq, generator=g)) if mix else None
    qs = [_rounded(torch.randn(n, Hq, hd, generator=g), dtype) for n in lengths]
    ks = [_rounded(torch.randn(n, G, hd, generator=g), dtype) for n in lengths]
    vs = [_rounded(torch.randn(n, G, vd, generator=g), dtype) for n in lengths]
    scale = 1.5 / math.sqrt(hd)
    cache = Paged(ks, vs, page, dtype, pool=pool, seed=2)
    cache.fill_pooled(lengths)
    rows = [(r, p) for r, n in enumerate(lengths) for p in range(n)]
    got = _attend(cache, torch.cat(qs), rows, scale, window, dtype, softcap=cap, talk=None if talk is None else talk.to(DEV))
    want = torch.cat([P.pooled_rows(q, k, v, window, pool, scale, cap, talk) for q, k, v in zip(qs, ks, vs)])
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


def test_block_means_are_taken_from_the_pages():
    """The mean key and value of every whole block, as the pages hold them (bfloat16 roundings included), at the
    row ``block`` of the pooled pages; a block that is not whole leaves nothing."""
    g = torch.Generator().manual_seed(5)
    for dtype, pool, page in ((torch.float32, 3, 4), (torch.bfloat16, 5, 8), (torch.float32, 1, 4), (torch.bfloat16, 16, 16)):
        lengths = [pool - 1 if pool > 1 else 1, 4 * pool + 2, 57]
        ks = [_rounded(torch.randn(n, 2, 24, generator=g), dtype) for n in lengths]
        vs = [_rounded(torch.randn(n, 2, 40, generator=g), dtype) for n in lengths]
        cache = Paged(ks, vs, page, dtype, pool=pool, seed=3)
        before = cache.kp.clone()
        cache.fill_pooled(lengths)
        torch.cuda.synchronize()
        table = cache.ptable.cpu()
        written = torch.zeros(cache.kp.shape[0], page, dtype=torch.bool)
        for r, n in enumerate(lengths):
            for b in range(n // pool):
                pg, slot = int(table[r, b // page]), b % page
                written[pg, slot] = True
                wk = ks[r][b * pool:(b + 1) * pool].mean(0)
                wv = vs[r][b * pool:(b + 1) * pool].mean(0)
                tol = 1e-6 if dtype == torch.float32 else 1e-2
                assert torch.allclose(cache.kp[pg, :, slot].float().cpu(), wk, atol=tol, rtol=tol)
                assert torch.allclose(cache.vp[pg, :, slot].float().cpu(), wv, atol=tol, rtol=tol)
        untouched = ~written.to(DEV)
        assert torch.equal(cache.kp.transpose(1, 2)[untouched], before.transpose(1, 2)[untouched])


# ---- one key that outweighs all others -----------------------------------------------------------------------
def _standout(n, G, hd, vd, where, g, big=40.0):
    """Keys and values of one sequence of ``n`` tokens: small random keys, and at the positions ``where`` a key
    ``big * e`` (``e`` a fixed unit direction) whose value is a vector of 100s; queries are ``e``."""
    e = torch.zeros(hd)
    e[1] = 1.0
    k = 0.05 * torch.randn(n, G, hd, generator=g)
    v = torch.randn(n, G, vd, generator=g)
    for j in where:
        k[j] = big * e
        v[j] = 100.0
    return e, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,page", [(7, 4), (16, 16), (33, 16), (64, 8), (100, 16)])
def test_a_key_at_the_windows_edge(window, page, dtype):
    """The standout key is read at distance window - 1 and not at distance window, wherever the key sits on its
    page (first slot, last slot) and whether the queries come as a prompt's rows or as single tokens."""
    g = torch.Generator().manual_seed(window)
    Hq, G, hd, vd, n = 4, 2, 32, 16, 3 * window + 2 * page + 5
    for j in {0, page - 1, page, 2 * page - 1, window, n - window - 1}:
        e, k, v = _standout(n, G, hd, vd, [j], g)
        cache = Paged([_rounded(k, dtype)], [_rounded(v, dtype)], page, dtype, seed=j)
        inside, outside = j + window - 1, j + window
        rows = [(0, p) for p in (j, inside, outside) if p < n]
        q = e.expand(len(rows), Hq, hd).contiguous()
        as_prompt = _attend(cache, q, rows, 1.0, window, dtype)
        singles = torch.cat([_attend(cache, q[i:i + 1], rows[i:i + 1], 1.0, window, dtype) for i in range(len(rows))])
        for got in (as_prompt, singles):
            assert float((got[0] - 100.0).abs().max()) < 1.0                   # the key itself
            if inside < n:
                assert float((got[1] - 100.0).abs().max()) < 1.0, (j, "just inside")
            if outside < n:
                assert float(got[len(rows) - 1].abs().max()) < 10.0, (j, "just outside")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,pool,page", [(6, 4, 4), (16, 16, 16), (9, 5, 8), (20, 3, 16), (5, 12, 4)])
def test_a_key_in_a_pooled_block(window, pool, page, dtype):
    """A block whose keys all stand out: its mean is read from the position ``last of the block + window`` on and
    not one token earlier; between leaving the window and that position its tokens are not read at all; a key
    hundreds of tokens back is still read through its block."""
    g = torch.Generator().manual_seed(window * pool)
    Hq, G, hd, vd = 2, 1, 16, 8
    n = 13 * pool + window + 3
    for b in (0, 1, 7):
        block = list(range(b * pool, (b + 1) * pool))
        e, k, v = _standout(n, G, hd, vd, block, g)
        cache = Paged([_rounded(k, dtype)], [_rounded(v, dtype)], page, dtype, pool=pool, seed=b)
        cache.fill_pooled([n])
        first, last = block[0], block[-1]
        seen_from = last + window
        places = {"in the window": first + window - 1, "just seen": seen_from, "far": n - 1}
        want = P.pooled_rows(e.expand(n, Hq, hd), _rounded(k, dtype), _rounded(v, dtype), window, pool, 1.0, 0.0, None)
        for what, p in places.items():
            got = _attend(cache, e.expand(1, Hq, hd).contiguous(), [(0, p)], 1.0, window, dtype)
            assert torch.allclose(got[0], want[p], atol=0.05, rtol=0.02), (what, b)
            if what in ("just seen", "far"):
                assert float((got - 100.0).abs().max()) < 1.0, (what, b)
        if pool == 1:
            continue
        # only the block's first token stands out: once it has left the window it is not read at all until the
        # block is whole and read as a mean
        e, k, v = _standout(n, G, hd, vd, [first], g, big=400.0)
        cache = Paged([_rounded(k, dtype)], [_rounded(v, dtype)], page, dtype, pool=pool, seed=b + 10)
        cache.fill_pooled([n])
        want = P.pooled_rows(e.expand(n, Hq, hd), _rounded(k, dtype), _rounded(v, dtype), window, pool, 1.0, 0.0, None)
        for what, p in {"last in the window": first + window - 1, "gap starts": first + window, "gap ends": seen_from - 1,
                        "mean": seen_from}.items():
            got = _attend(cache, e.expand(1, Hq, hd).contiguous(), [(0, p)], 1.0, window, dtype)
            assert torch.allclose(got[0], want[p], atol=0.05, rtol=0.02), (what, b)
            if what.startswith("gap"):
                assert float(got.abs().max()) < 10.0, (what, b)
            elif what == "last in the window":
                assert float((got - 100.0).abs().max()) < 1.0, (what, b)
            else:
                assert float(got.abs().max()) > 100.0 / pool - 5.0, (what, b)


def test_the_first_tokens_and_the_sink_alone():
    """Position 0 reads itself only: with a sink its weight is exp(s) / (exp(s) + exp(sink)), below 1."""
    g = torch.Generator().manual_seed(0)
    Hq, G, hd, vd = 2, 2, 8, 8
    q, k, v = torch.randn(3, Hq, hd, generator=g), torch.randn(3, G, hd, generator=g), torch.randn(3, G, vd, generator=g)
    sink = torch.tensor([0.3, -1.2])
    cache = Paged([k], [v], 4, torch.float32)
    got = _attend(cache, q[:1], [(0, 0)], 0.5, 5, torch.float32, sink=sink.to(DEV))
    for h in range(Hq):
        s = float(q[0, h] @ k[0, h]) * 0.5
        w = math.exp(s) / (math.exp(s) + math.exp(float(sink[h])))
        assert torch.allclose(got[0, h], w * v[0, h], atol=1e-5)
