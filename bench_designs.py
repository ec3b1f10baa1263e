"""``bench.py --design guravik`` / ``--design tirizen`` / ``--design tarulix`` / ``--design puvolix``: another decoder beside the MiniMax-M3 decoder at equal sizes.

For a few sizes that resemble a real model's layers (seeded random weights, bfloat16): one prompt of
``--prompt-len`` tokens as one step (tokens a second) and decode steps of ``--batch`` requests at that
context (tokens a second), each model through the same engine, step function and captured decode steps.
"Equal size": the same width, layer count and vocabulary, as many attention heads of the same size, and a
routed feed-forward whose two active experts are as wide together as the dense feed-forward.

Then the new design's kernels alone, each beside the kernel of the softmax-attention model that does the
like job, as fractions of the same peaks (measured if MEASURED_PEAKS.json is there, else the fallback):
attention over a prompt (flops / time / tensor peak) and over single tokens (cache bytes / time / copy
bandwidth), and the recurrence (state bytes / time / copy bandwidth for single tokens; tokens a second and
float32 flops a second for a prompt, where it is a chain in time and has no tensor-core form here).
Times are medians of CUDA-event intervals after warm-up; decode kernels run back to back in a CUDA graph on
caches of several layers, larger than L2.

``--design tirizen``: the same two model measurements for the Tirizen decoder (layers: attention with routed
experts, gated linear attention with routed experts, attention that reads the first layer's keys and values;
three residual streams), whose attention and expert products run on the SAME kernels as MiniMax-M3's at these
sizes; alone are measured the kernels that are its own: the gated linear recurrence beside Guravik's delta-rule
recurrence (the like kernel), and the launch between two sublayers (streams written back, read and normed)
beside the adding RMS norm, both as bytes / time / copy bandwidth.

``--design tarulix``: the same two model measurements for the Tarulix decoder (layers: two windowed attentions with
distance bias, sink and blended values, then a rotary windowed attention with pooled blocks beside a selective scan;
routed, pass-through and shared experts).  Alone: ``window_attention`` in both forms over a prompt (flops / time /
tensor peak) and over single tokens deep in a context (visible cache bytes / time / copy bandwidth) beside the
softmax-attention kernels of MiniMax-M3, and ``selective_scan`` beside Tirizen's gated linear recurrence.

``--design puvolix``: the Puvolix decoder (every layer a softmax attention with 32-bit weights beside a gated delta
rule; a dense layer with biases first, then routed experts with a shared expert; norms in groups; a depth-weighted
stream) beside Tarulix, the closest existing model (a parallel attention and recurrence, output norms, routed and
shared experts), and MiniMax-M3, all at equal sizes.  Alone: the attention kernels in the form Puvolix runs them
(no window) beside Tarulix's biased form and MiniMax-M3's; ``gated_delta`` beside Guravik's ``delta_rule`` (the like
chain in time) and Tirizen's ``gla``; the launch between two sublayers (``grouped_normed_add`` with branch norms,
and with the depth-weighted sum) beside ``normed_add_rmsnorm``.
"""

from __future__ import annotations

import json
import math
import random
import statistics
import sys
import time

SIZES = {
    # width, layers (one latent-attention layer with a feed-forward, then two delta-rule layers without), heads ...
    "w2048": dict(width=2048, groups=2, vocab=32000, ff=5632, attn_heads=16, dim=128, rot=64, vdim=128, q_rank=768,
                  kv_rank=256, delta_heads=32, delta_dim=64),
    "w4096": dict(width=4096, groups=2, vocab=32000, ff=11008, attn_heads=32, dim=128, rot=64, vdim=128, q_rank=1536,
                  kv_rank=512, delta_heads=64, delta_dim=64),
}


def guravik_raw(s: dict) -> dict:
    latent = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": s["ff"]},
              "mixer": {"heads": s["attn_heads"], "dim": s["dim"], "rot_dim": s["rot"], "vdim": s["vdim"], "q_rank": s["q_rank"],
                        "kv_rank": s["kv_rank"], "scale": 1.0 / math.sqrt(s["dim"] + s["rot"]),
                        "rot": {"base": 1e6, "dims": s["rot"]}}}
    delta = {"type": "general_delta", "mixer": {"heads": s["delta_heads"], "dim": s["delta_dim"]}, "mlp": None}
    return {"architecture": "Guravik", "vocab": s["vocab"], "width": s["width"], "layers": [latent, delta, delta] * s["groups"],
            "canon": {"taps": 3}, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "loop": {"start": 0, "stop": 0, "times": 1}}


TIRIZEN_SIZES = {
    "w2048": dict(width=2048, groups=2, vocab=32000, ff=5632, attn_heads=16, dim=128, gla_heads=32, gla_dim=64, streams=3),
    "w4096": dict(width=4096, groups=2, vocab=32000, ff=11008, attn_heads=32, dim=128, gla_heads=64, gla_dim=64, streams=3),
}


def tirizen_raw(s: dict) -> dict:
    """Per group of three layers: attention, gated linear attention, attention on the first one's keys and values;
    every layer with 8 routed experts of which 2 are active, together as wide as ``ff``."""
    moe = {"kind": "moe", "expert": {"ff": s["ff"] // 2}, "router": {"experts": 8, "top": 2}}
    layers = []
    for g in range(s["groups"]):
        attn = {"heads": s["attn_heads"], "kv_heads": max(1, s["attn_heads"] // 4), "dim": s["dim"], "vdim": s["dim"],
                "scale": 1.0 / math.sqrt(s["dim"]), "q_temp": {"coef": 0.25, "every": 512}}
        layers += [{"type": "attention", "mixer": dict(attn), "mlp": moe},
                   {"type": "gla", "mixer": {"heads": s["gla_heads"], "dim": s["gla_dim"], "vdim": s["gla_dim"], "tau": 8.0,
                                             "decay_rank": 32}, "mlp": moe},
                   {"type": "attention", "mixer": dict(attn, kv_from=3 * g), "mlp": moe}]
    return {"architecture": "Tirizen", "vocab": s["vocab"], "width": s["width"], "layers": layers, "streams": s["streams"],
            "residual_mult": 0.8, "embedding": {"scale": 1.0}, "logit_scale": 1.0, "norm": {"eps": 1e-5},
            "max_positions": 8192}


TARULIX_SIZES = {
    "w2048": dict(width=2048, groups=2, vocab=32000, ff=5632, attn_heads=16, dim=128, window=1024, pool=64, rot=64, inner=4096,
                  state=16, dt_rank=128, taps=4),
    "w4096": dict(width=4096, groups=2, vocab=32000, ff=11008, attn_heads=32, dim=128, window=1024, pool=64, rot=64, inner=8192,
                  state=16, dt_rank=256, taps=4),
}


PUVOLIX_SIZES = {
    "w2048": dict(width=2048, groups=2, vocab=32000, ff=5632, attn_heads=16, dim=128, rot=64, delta_heads=16, delta_groups=8,
                  delta_dim=128, norm_groups=8, window=1024, pool=64, inner=4096, state=16, dt_rank=128, taps=4),
    "w4096": dict(width=4096, groups=2, vocab=32000, ff=11008, attn_heads=32, dim=128, rot=64, delta_heads=32, delta_groups=16,
                  delta_dim=128, norm_groups=8, window=1024, pool=64, inner=8192, state=16, dt_rank=256, taps=4),
}


def puvolix_raw(s: dict) -> dict:
    """Six layers, each a softmax attention (a quarter as many kv heads, half the head rotated, rescaled frequencies,
    convolutions of 4 taps) beside a gated delta rule (heads of 128 x 128 in groups of two, convolutions of 4 taps);
    the first layer's feed-forward dense with biases, the others 8 routed experts of which 2 are chosen and a shared
    expert, together as wide as ``ff``."""
    moe = {"kind": "moe", "expert": {"ff": 3 * s["ff"] // 8, "limit": 7.0}, "router": {"experts": 8, "top": 2},
           "shared": {"ff": s["ff"] // 4, "limit": 7.0}}
    left = {"heads": s["attn_heads"], "kv_heads": max(1, s["attn_heads"] // 4), "dim": s["dim"], "vdim": s["dim"], "conv": 4,
            "scale": 1.0 / math.sqrt(s["dim"]),
            "rot": {"dims": s["rot"], "base": 5e5, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": s["delta_heads"], "kv_heads": s["delta_groups"], "dim": s["delta_dim"], "vdim": s["delta_dim"], "conv": 4}
    layers = [{"type": "parallel", "mixer": {"left": dict(left), "right": dict(right)},
               "mlp": {"kind": "dense", "ff": s["ff"]} if i == 0 else moe} for i in range(3 * s["groups"])]
    return {"architecture": "Puvolix", "vocab": s["vocab"], "width": s["width"], "layers": layers,
            "norm": {"eps": 1e-5, "groups": s["norm_groups"]}, "logit_softcap": 30.0}


def tarulix_raw(s: dict) -> dict:
    """Per group of three layers: two windowed attention layers with distance bias, sink and blended values, then a
    rotary windowed attention with pooled blocks beside a selective scan; every layer with 8 routed experts and 2
    pass-through experts of which 2 are chosen, and a shared expert: two routed experts and the shared one are
    together as wide as ``ff``."""
    moe = {"kind": "moe", "expert": {"ff": 3 * s["ff"] // 8}, "router": {"experts": 8, "identity": 2, "top": 2},
           "shared": {"ff": s["ff"] // 4}}
    heads = {"heads": s["attn_heads"], "kv_heads": max(1, s["attn_heads"] // 4), "dim": s["dim"], "vdim": s["dim"],
             "scale": 1.0 / math.sqrt(s["dim"])}
    attn = dict(heads, mask={"size": s["window"]}, bias_max=4 * s["window"], v_mix=True)
    left = dict(heads, mask={"size": s["window"], "pool": s["pool"]}, rot={"dims": s["rot"], "base": 5e5}, softcap=20.0)
    right = {"inner": s["inner"], "state": s["state"], "dt_rank": s["dt_rank"], "conv": s["taps"]}
    layers = []
    for _ in range(s["groups"]):
        layers += [{"type": "attention", "mixer": dict(attn), "mlp": moe}, {"type": "attention", "mixer": dict(attn), "mlp": moe},
                   {"type": "parallel", "mixer": {"left": dict(left), "right": dict(right), "left_scale": 0.75, "right_scale": 1.1},
                    "mlp": moe}]
    return {"architecture": "Tarulix", "vocab": s["vocab"], "width": s["width"], "layers": layers, "norm": {"eps": 1e-5}}


def minimax_raw(s: dict) -> dict:
    return dict(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"] // 2, num_hidden_layers=3 * s["groups"],
                num_attention_heads=s["attn_heads"], num_key_value_heads=max(1, s["attn_heads"] // 4), head_dim=128, rotary_dim=64,
                rope_theta=1e6, use_qk_norm=True, qk_norm_type="per_layer", num_local_experts=8, num_experts_per_tok=2,
                use_routing_bias=True, rms_norm_eps=1e-5, tie_word_embeddings=False, architectures=["MiniMaxM3ForCausalLM"],
                model_type="minimax_m3")


def _model_numbers(cfg, prompt_len: int, batch: int, steps: int, warmup: int) -> dict:
    import torch
    from quanta_b200 import kernels
    from quanta_b200.engine.model import random_model
    from quanta_b200.engine.step import Engine, StepEntry
    model = random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    params = sum(p.numel() for part in model.parts() for p in vars(part).values() if isinstance(p, torch.Tensor))
    page, context = 16, prompt_len + warmup + steps + 16
    eng = Engine(model, num_pages=(batch + 1) * -(-context // page), page_size=page, max_requests=batch + 1)
    rng = random.Random(0)
    V = model.spec.vocab_size
    toks = lambda n: [rng.randrange(V) for _ in range(n)]  # noqa: E731
    pre = []
    for i in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p = toks(prompt_len)
        torch.cuda.synchronize()
        a.record()
        eng.step([StepEntry(("p", i), p, (prompt_len - 1,))], end=[("p", i)])
        b.record()
        torch.cuda.synchronize()
        pre.append(a.elapsed_time(b))
    pre_ms = statistics.median(pre[2:])
    rids = [("d", i) for i in range(batch)]
    for rid in rids:
        eng.step([StepEntry(rid, toks(prompt_len), ())])
    out = torch.empty(batch, dtype=torch.int32, device="cuda:0")
    kernels.LAUNCHES = 0
    evs = []
    for i in range(warmup + steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lg = eng.step([StepEntry(rid, [rng.randrange(V)], (0,)) for rid in rids])
        kernels.sample_rows(lg, None, None, out)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    eng.check()
    dec_ms = statistics.fmean(a.elapsed_time(b) for a, b in evs[warmup:])
    launches = kernels.LAUNCHES // (warmup + steps)
    stats = eng.stats()
    del eng, model
    torch.cuda.empty_cache()
    return {"parameters_m": round(params / 1e6, 1), "prefill_tokens": prompt_len, "prefill_ms": round(pre_ms, 3),
            "prefill_tok_s": round(prompt_len / pre_ms * 1e3, 1), "decode_batch": batch, "decode_ms": round(dec_ms, 4),
            "decode_tok_s": round(batch / dec_ms * 1e3, 1), "launches_per_decode_step": int(launches),
            "graph_replays": stats["graph_replays"]}


# ---- kernels alone -------------------------------------------------------------------------------------
def latent_prefill(tokens: int, heads: int, C: int, R: int, page: int = 16) -> dict:
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    pages = -(-tokens // page)
    table = torch.randperm(pages, dtype=torch.int32).view(1, -1).to(dev)
    cache = torch.randn(pages, 1, page, C + R, device=dev, dtype=torch.bfloat16)
    q_lat = torch.randn(heads, tokens, C, device=dev)
    q_rot = torch.randn(tokens, heads, R, device=dev)
    sink = torch.zeros(heads, device=dev)
    out = torch.empty(heads, tokens, C, device=dev, dtype=torch.bfloat16)
    pos = torch.arange(tokens, dtype=torch.int32, device=dev)
    req = torch.zeros(tokens, dtype=torch.int32, device=dev)
    st = k.new_status(dev)
    starts = torch.tensor([0, tokens], dtype=torch.int32, device=dev)
    ms = bk.timed(lambda: k.latent_attend(q_lat, q_rot, cache, sink, out, pos, req, table, 0.1, 1, st, req_start=starts), n=5, warm=2)
    keys = tokens * (tokens + 1) // 2
    flops = (2.0 * (C + R) + 2.0 * C) * heads * keys
    return {"kernel": "latent_attend (prompt)", "tokens": tokens, "heads": heads, "latent": C, "rot": R, "ms": round(ms, 3),
            "TFLOP/s": round(flops / ms / 1e9, 2)}


def latent_decode(batch: int, context: int, heads: int, C: int, R: int, page: int = 16) -> dict:
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    per = -(-context // page)
    layers = max(1, min(16, int(3e9 // (batch * per * page * (C + R) * 2))))
    caches = [torch.randn(batch * per, 1, page, C + R, device=dev, dtype=torch.bfloat16) for _ in range(layers)]
    table = torch.randperm(batch * per, dtype=torch.int32).view(batch, per).to(dev)
    q_lat = torch.randn(heads, batch, C, device=dev)
    q_rot = torch.randn(batch, heads, R, device=dev)
    sink = torch.zeros(heads, device=dev)
    out = torch.empty(heads, batch, C, device=dev, dtype=torch.bfloat16)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    req = torch.arange(batch, dtype=torch.int32, device=dev)
    st = k.new_status(dev)
    blocks = -(-batch * heads // k.LATENT_MMA_ROWS) if k.latent_attend_uses_tensor_cores(torch.bfloat16, C, R) else batch * -(-heads // 8)
    n_ranges = max(1, min(64, -(-296 // blocks), -(-context // 128)))
    starts = torch.arange(batch + 1, dtype=torch.int32, device=dev)

    def all_layers():
        for c in caches:
            k.latent_attend(q_lat, q_rot, c, sink, out, pos, req, table, 0.1, n_ranges, st, req_start=starts)
    ms = bk.timed_graph(all_layers, reps=1) / layers
    nbytes = batch * context * (C + R) * 2
    return {"kernel": "latent_attend + merge (single tokens)", "batch": batch, "context": context, "heads": heads, "latent": C,
            "rot": R, "ranges": n_ranges, "us": round(ms * 1e3, 2), "GB/s": round(nbytes / ms / 1e6, 1)}


def delta_rule(tokens_per_req: int, reqs: int, heads: int, D: int) -> dict:
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    T, HD = tokens_per_req * reqs, heads * D
    proj = torch.randn(T, 4 * HD, device=dev)
    wpre = torch.randn(T, HD, device=dev)
    a_b, w_b = torch.zeros(HD, device=dev), torch.zeros(HD, device=dev)
    layers = 1 if tokens_per_req > 1 else max(1, min(16, int(2e9 // (reqs * heads * D * D * 4))))
    states = [torch.zeros(reqs, heads, D, D, device=dev) for _ in range(layers)]
    out = torch.empty(T, heads, D, device=dev)
    starts = torch.arange(0, T + 1, tokens_per_req, dtype=torch.int32, device=dev)
    slots = torch.arange(reqs, dtype=torch.int32, device=dev)

    def all_layers():
        for s in states:
            k.delta_rule(proj, (0, HD, 2 * HD, 3 * HD), wpre, a_b, w_b, s, out, starts, slots, heads, D, math.exp(-0.5), 1e-6)
    ms = (bk.timed_graph(all_layers, reps=1) if tokens_per_req == 1 else bk.timed(all_layers, n=5, warm=2)) / layers
    state_bytes = 2 * reqs * heads * D * D * 4 + T * 5 * HD * 4
    return {"kernel": "delta_rule", "requests": reqs, "tokens_per_request": tokens_per_req, "heads": heads, "dim": D,
            "us": round(ms * 1e3, 2), "tokens/s": round(T / ms * 1e3, 1), "GB/s": round(state_bytes / ms / 1e6, 1),
            "fp32 TFLOP/s": round(8.0 * D * D * heads * T / ms / 1e9, 2)}


def gla(tokens_per_req: int, reqs: int, heads: int, D: int, E: int, rank: int = 16) -> dict:
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    T, HD, HE = tokens_per_req * reqs, heads * D, heads * E
    proj = torch.randn(T, 2 * HD + 2 * HE + rank, device=dev)
    w2 = torch.randn(HD, rank, device=dev, dtype=torch.bfloat16)
    bias = torch.full((HD,), 3.0, device=dev)
    layers = 1 if tokens_per_req > 1 else max(1, min(16, int(2e9 // (reqs * heads * D * E * 4))))
    states = [torch.zeros(reqs, heads, D, E, device=dev) for _ in range(layers)]
    out = torch.empty(T, heads, E, device=dev)
    starts = torch.arange(0, T + 1, tokens_per_req, dtype=torch.int32, device=dev)
    slots = torch.arange(reqs, dtype=torch.int32, device=dev)

    def all_layers():
        for s in states:
            k.gla(proj, (0, HD, 2 * HD), 2 * HD + 2 * HE, rank, w2, bias, s, out, starts, slots, heads, D, E, 16.0, D ** -0.5)
    ms = (bk.timed_graph(all_layers, reps=1) if tokens_per_req == 1 else bk.timed(all_layers, n=5, warm=2)) / layers
    nbytes = 2 * reqs * heads * D * E * 4 + T * (3 * HD + 2 * HE) * 4      # the state read and written; q, k, alpha, v, o
    return {"kernel": "gla (decay + chain)", "requests": reqs, "tokens_per_request": tokens_per_req, "heads": heads, "dim": D,
            "vdim": E, "us": round(ms * 1e3, 2), "tokens/s": round(T / ms * 1e3, 1), "GB/s": round(nbytes / ms / 1e6, 1),
            "fp32 TFLOP/s": round(4.0 * D * E * heads * T / ms / 1e9, 2)}


def streams_norm(tokens: int, S: int, H: int) -> dict:
    """The launch between two sublayers of a model with S residual streams, and the adding norm of a model with one."""
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    n = max(1, int(1.5e9 // (tokens * (2 * S + 1) * H * 4)))
    xs = [torch.randn(tokens, S, H, device=dev) for _ in range(n)]
    hs = [torch.randn(tokens, H, device=dev) for _ in range(n)]
    y = torch.randn(tokens, H, device=dev)
    mix, out_w, read_w = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev)
    w = torch.ones(H, device=dev)
    out = torch.empty(tokens, H, device=dev, dtype=torch.bfloat16)

    def many_streams():
        for x in xs:
            k.streams_mix_rmsnorm(x, y, mix, out_w, 0.7, read_w, w, 1e-5, out)

    def one_stream():
        for h in hs:
            k.add_rmsnorm(h, y, w, 1e-5, out)
    a = bk.timed_graph(many_streams, reps=1) / n
    b = bk.timed_graph(one_stream, reps=1) / n
    bytes_a, bytes_b = tokens * ((2 * S + 1) * H * 4 + H * 2), tokens * (3 * H * 4 + H * 2)
    return {"kernel": "streams_mix_rmsnorm", "tokens": tokens, "streams": S, "width": H, "us": round(a * 1e3, 2),
            "GB/s": round(bytes_a / a / 1e6, 1), "add_rmsnorm_us": round(b * 1e3, 2), "add_rmsnorm_GB/s": round(bytes_b / b / 1e6, 1)}


def run_tirizen(args) -> dict:
    import bench
    from quanta_b200.config import MiniMaxM3Config, TirizenConfig
    pk, pk_src = bench.peaks()
    clocks = bench.ClockSampler()
    clocks.start()
    models = {}
    for name, s in TIRIZEN_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        t0 = time.time()
        t = _model_numbers(TirizenConfig.from_dict(tirizen_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        m = _model_numbers(MiniMaxM3Config.from_dict(minimax_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        models[name] = {"sizes": s, "tirizen": t, "minimax_m3": m}
        print(f"[bench] {name}: tirizen {t}\n[bench] {name}: minimax_m3 {m} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    s = TIRIZEN_SIZES["w2048"]
    T, B, hbm = args.prompt_len, args.batch, pk["hbm_gbs"] * 1e9
    gp, gd = gla(T, 1, s["gla_heads"], s["gla_dim"], s["gla_dim"]), gla(1, B, s["gla_heads"], s["gla_dim"], s["gla_dim"])
    dp, dd = delta_rule(T, 1, s["gla_heads"], s["gla_dim"]), delta_rule(1, B, s["gla_heads"], s["gla_dim"])
    sn_p, sn_d = streams_norm(T, s["streams"], s["width"]), streams_norm(B, s["streams"], s["width"])
    for r in (gp, gd, dp, dd, sn_p, sn_d):
        r["frac_of_copy_bandwidth"] = round(r["GB/s"] * 1e9 / hbm, 4)
    for r in (sn_p, sn_d):
        r["add_rmsnorm_frac_of_copy_bandwidth"] = round(r["add_rmsnorm_GB/s"] * 1e9 / hbm, 4)
    kernels_alone = {"recurrence_prompt": {"tirizen": gp, "guravik": dp}, "recurrence_single_tokens": {"tirizen": gd, "guravik": dd},
                     "between_sublayers_prompt": sn_p, "between_sublayers_single_tokens": sn_d}
    for k_, v in kernels_alone.items():
        print(f"[bench] {k_}: {v}", file=sys.stderr, flush=True)
    first = next(iter(models.values()))["tirizen"] if models else {}
    return {"metric": f"Tirizen decode tokens/s (batch {args.batch}, {args.prompt_len}-token prompts) beside MiniMax-M3 at equal sizes",
            "value": first.get("decode_tok_s"), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": first.get("decode_ms"), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)", "design": "tirizen", "models": models,
            "kernels": kernels_alone, "peaks": {**pk, "source": pk_src}, "clocks": clocks.stop(),
            "gpu_launches": first.get("launches_per_decode_step", 0) * args.steps, "impl": "ours"}


def window_attn(tokens_per_req: int, reqs: int, context: int, nq: int, nkv: int, hd: int, window: int, kind: str,
                pool: int = 64, page: int = 16) -> dict:
    """``window_attention`` alone: ``reqs`` requests whose last ``tokens_per_req`` tokens (ending at ``context``) are
    the step.  ``kind`` "biased": distance bias and sink; "pooled": score cap, pooled blocks and mixed head weights
    (with the second launch that mixes).  Flops count ``4 * head_dim`` a (query head, visible key), pooled rows too;
    bytes count the visible keys and values once a request."""
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    per = -(-context // page)
    single = tokens_per_req == 1
    layers = 1 if not single else max(1, min(16, int(3e9 // (2 * reqs * per * nkv * page * hd * 2))))
    caches = [(torch.randn(reqs * per, nkv, page, hd, device=dev, dtype=torch.bfloat16),
               torch.randn(reqs * per, nkv, page, hd, device=dev, dtype=torch.bfloat16)) for _ in range(layers)]
    table = torch.randperm(reqs * per, dtype=torch.int32).view(reqs, per).to(dev)
    T = tokens_per_req * reqs
    q = torch.randn(T, nq, hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.arange(context - tokens_per_req, context, dtype=torch.int32, device=dev).repeat(reqs)
    req = torch.arange(reqs, dtype=torch.int32, device=dev).repeat_interleave(tokens_per_req)
    st = k.new_status(dev)
    extras = {}
    if kind == "biased":
        extras = dict(dist_bias=torch.randn(window, nq, device=dev), sink=torch.zeros(nq, device=dev))
    else:
        rows = -(-context // pool)
        ppp = -(-rows // page)
        extras = dict(softcap=20.0, pool=pool, pooled_k=torch.randn(reqs * ppp, nkv, page, hd, device=dev, dtype=torch.bfloat16),
                      pooled_v=torch.randn(reqs * ppp, nkv, page, hd, device=dev, dtype=torch.bfloat16),
                      pool_table=torch.randperm(reqs * ppp, dtype=torch.int32).view(reqs, ppp).to(dev),
                      talk=torch.eye(nq, device=dev) + 0.1 * torch.randn(nq, nq, device=dev),
                      scratch=torch.empty(T, nq, nkv, hd, device=dev))

    def all_layers():
        for kc, vc in caches:
            k.window_attention(q, kc, vc, out, pos, req, table, hd ** -0.5, window, st, n_requests=reqs, **extras)
    ms = (bk.timed_graph(all_layers, reps=1) if single else bk.timed(all_layers, n=5, warm=2)) / layers
    k.raise_on_status(st.cpu())
    seen = 0
    for p_ in range(context - tokens_per_req, context):
        seen += min(p_ + 1, window) + (max(0, (p_ - window + 1) // pool) if kind == "pooled" else 0)
    flops = 4.0 * hd * nq * seen * reqs
    first = max(0, context - tokens_per_req - window + 1)
    rows_read = (context - first) + (max(0, (context - window) // pool) if kind == "pooled" else 0)
    nbytes = reqs * rows_read * nkv * hd * 2 * 2
    return {"kernel": f"window_attention ({kind})", "requests": reqs, "tokens_per_request": tokens_per_req, "context": context,
            "q_heads": nq, "kv_heads": nkv, "head_dim": hd, "window": window, "layers": layers, "us": round(ms * 1e3, 2),
            "TFLOP/s": round(flops / ms / 1e9, 2), "GB/s": round(nbytes / ms / 1e6, 1)}


def plain_attn(tokens_per_req: int, reqs: int, context: int, nq: int, nkv: int, hd: int, page: int = 16) -> dict:
    """The attention as Puvolix runs it: ``window_attention`` over all keys, no extras; portions on the tensor cores
    with the weights in two bfloat16 parts, single tokens with their keys cut into ranges and a join (32-bit
    arithmetic).  Flops count ``4 * head_dim`` a (query head, visible key); bytes the visible keys and values once."""
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    per = -(-context // page)
    single = tokens_per_req == 1
    layers = 1 if not single else max(1, min(16, int(3e9 // (2 * reqs * per * nkv * page * hd * 2))))
    caches = [(torch.randn(reqs * per, nkv, page, hd, device=dev, dtype=torch.bfloat16),
               torch.randn(reqs * per, nkv, page, hd, device=dev, dtype=torch.bfloat16)) for _ in range(layers)]
    table = torch.randperm(reqs * per, dtype=torch.int32).view(reqs, per).to(dev)
    T = tokens_per_req * reqs
    q = torch.randn(T, nq, hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.arange(context - tokens_per_req, context, dtype=torch.int32, device=dev).repeat(reqs)
    req = torch.arange(reqs, dtype=torch.int32, device=dev).repeat_interleave(tokens_per_req)
    st = k.new_status(dev)
    n_split = max(1, min(-(-2048 // (T * nkv)), -(-context // 32), 256))      # as parts/attention.py chooses it

    def all_layers():
        for kc, vc in caches:
            k.window_attention(q, kc, vc, out, pos, req, table, hd ** -0.5, 0, st, n_split=n_split, n_requests=reqs)
    ms = (bk.timed_graph(all_layers, reps=1) if single else bk.timed(all_layers, n=5, warm=2)) / layers
    k.raise_on_status(st.cpu())
    seen = sum(p_ + 1 for p_ in range(context - tokens_per_req, context))
    flops = 4.0 * hd * nq * seen * reqs
    nbytes = reqs * context * nkv * hd * 2 * 2
    return {"kernel": "window_attention (all keys, no extras)", "requests": reqs, "tokens_per_request": tokens_per_req,
            "context": context, "q_heads": nq, "kv_heads": nkv, "head_dim": hd, "layers": layers, "ranges": n_split if single else 1,
            "us": round(ms * 1e3, 2), "TFLOP/s": round(flops / ms / 1e9, 2), "GB/s": round(nbytes / ms / 1e6, 1)}


def gated_delta(tokens_per_req: int, reqs: int, heads: int, groups: int, D: int, DV: int) -> dict:
    """``gated_delta`` alone (preparation + chain).  Bytes: the state read and written, and per token the rows read
    (q, k, v, the two pre-activations), the unit q and k written and read, and the output."""
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    T = tokens_per_req * reqs
    C = 2 * groups * D + heads * DV
    qkv = torch.randn(T, C, device=dev)
    ab = torch.randn(T, 2 * heads, device=dev)
    A_log, dt_b = torch.zeros(heads, device=dev), torch.zeros(heads, device=dev)
    layers = 1 if tokens_per_req > 1 else max(1, min(16, int(2e9 // (reqs * heads * D * DV * 4))))
    states = [torch.zeros(reqs, heads, D, DV, device=dev) for _ in range(layers)]
    out = torch.empty(T, heads, DV, device=dev)
    starts = torch.arange(0, T + 1, tokens_per_req, dtype=torch.int32, device=dev)
    slots = torch.arange(reqs, dtype=torch.int32, device=dev)

    def all_layers():
        for s in states:
            k.gated_delta(qkv, ab, 0, heads, A_log, dt_b, s, out, starts, slots, heads, groups, D, DV, D ** -0.5, 1e-6)
    ms = (bk.timed_graph(all_layers, reps=1) if tokens_per_req == 1 else bk.timed(all_layers, n=5, warm=2)) / layers
    nbytes = 2 * reqs * heads * D * DV * 4 + T * (C + 2 * heads + 4 * groups * D + heads * DV) * 4
    return {"kernel": "gated_delta (preparation + chain)", "requests": reqs, "tokens_per_request": tokens_per_req, "heads": heads,
            "groups": groups, "dim": D, "value_dim": DV, "layers": layers, "us": round(ms * 1e3, 2),
            "tokens/s": round(T / ms * 1e3, 1), "GB/s": round(nbytes / ms / 1e6, 1),
            "fp32 TFLOP/s": round(7.0 * D * DV * heads * T / ms / 1e9, 2)}


def between_sublayers(tokens: int, H: int, groups: int, depth: int) -> dict:
    """One launch between two sublayers, bytes / time: ``grouped_normed_add`` with two normed branches and a norm in
    groups (the mixer's output joins the stream, the feed-forward reads it), the same with routed slots, a shared
    expert and the depth-weighted sum over ``depth`` earlier results, and ``normed_add_rmsnorm`` (one norm over the
    row, two addends) for comparison."""
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    h = torch.randn(tokens, H, device=dev)
    a, b = torch.randn(tokens, H, device=dev), torch.randn(tokens, H, device=dev)
    slots = torch.randn(tokens, 2, H, device=dev)
    g1, g2, g = (torch.rand(H, device=dev) + 0.5 for _ in range(3))
    out = torch.empty(tokens, H, device=dev, dtype=torch.bfloat16)
    hist = torch.randn(depth + 1, tokens, H, device=dev)
    w = torch.rand(depth + 1, device=dev)
    small = tokens <= 64
    run = (lambda f: bk.timed_graph(f, reps=20)) if small else (lambda f: bk.timed(f, n=10, warm=3))
    t_mix = run(lambda: k.grouped_normed_add(h, y=a, y_scale=0.5, y_gain=g1, extra=b, extra_scale=0.5, extra_gain=g2, branch_eps=1e-5,
                                             gain=g, groups=groups, gain_eps=1e-5, out=out))
    t_depth = run(lambda: k.grouped_normed_add(h, y=slots, extra=b, gain=g, groups=groups, gain_eps=1e-5, history=hist,
                                               n_history=depth, history_weights=w))
    t_old = run(lambda: k.normed_add_rmsnorm(h, a, g, 1e-5, None, 0.0, out, y_scale=0.5, extra=b, extra_scale=0.5))
    row = H * 4
    by = {"branches + group norm": tokens * (4 * row + H * 2), "slots + shared + depth sum": tokens * ((5 + depth + 1) * row),
          "normed_add_rmsnorm": tokens * (4 * row + H * 2)}
    res = {"tokens": tokens, "width": H, "groups": groups, "depth": depth}
    for name, ms in (("branches + group norm", t_mix), ("slots + shared + depth sum", t_depth), ("normed_add_rmsnorm", t_old)):
        res[name] = {"us": round(ms * 1e3, 2), "GB/s": round(by[name] / ms / 1e6, 1)}
    return res


def run_puvolix(args) -> dict:
    import bench
    import bench_kernels as bk
    from quanta_b200.config import MiniMaxM3Config, PuvolixConfig, TarulixConfig
    pk, pk_src = bench.peaks()
    clocks = bench.ClockSampler()
    clocks.start()
    models = {}
    for name, s in PUVOLIX_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        t0 = time.time()
        p = _model_numbers(PuvolixConfig.from_dict(puvolix_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        t = _model_numbers(TarulixConfig.from_dict(tarulix_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        m = _model_numbers(MiniMaxM3Config.from_dict(minimax_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        models[name] = {"sizes": s, "puvolix": p, "tarulix": t, "minimax_m3": m}
        print(f"[bench] {name}: puvolix {p}\n[bench] {name}: tarulix {t}\n[bench] {name}: minimax_m3 {m} ({time.time() - t0:.0f} s)",
              file=sys.stderr, flush=True)
    s = PUVOLIX_SIZES["w2048"]
    T, B = args.prompt_len, args.batch
    tensor, hbm = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    Hq, Hk, hd = s["attn_heads"], max(1, s["attn_heads"] // 4), s["dim"]
    pp, pd = plain_attn(T, 1, T, Hq, Hk, hd), plain_attn(1, B, T, Hq, Hk, hd)
    tp, td = window_attn(T, 1, T, Hq, Hk, hd, s["window"], "biased"), window_attn(1, B, 4 * T, Hq, Hk, hd, s["window"], "biased")
    sp, sd = bk.attn_span(T, 0, Hq, Hk, hd, 16), bk.attn_decode(B, T, Hq, Hk, hd, 16)
    for r in (pp, tp, sp):
        r["frac_of_tensor_peak"] = round(r["TFLOP/s"] * 1e12 / tensor, 4)
    for r in (pd, td, sd):
        r["frac_of_copy_bandwidth"] = round(r["GB/s"] * 1e9 / hbm, 4)
    H_, G_, D_ = s["delta_heads"], s["delta_groups"], s["delta_dim"]
    gp, gd, gd64 = gated_delta(T, 1, H_, G_, D_, D_), gated_delta(1, B, H_, G_, D_, D_), gated_delta(1, 64, H_, G_, D_, D_)
    dp, dd = delta_rule(T, 1, H_, D_), delta_rule(1, B, H_, D_)
    lp, ld = gla(T, 1, H_, D_, D_), gla(1, B, H_, D_, D_)
    for r in (gp, gd, gd64, dp, dd, lp, ld):
        r["frac_of_copy_bandwidth"] = round(r["GB/s"] * 1e9 / hbm, 4)
    bp, bd = between_sublayers(T, s["width"], s["norm_groups"], 6), between_sublayers(B, s["width"], s["norm_groups"], 6)
    for r in (bp, bd):
        for v in r.values():
            if isinstance(v, dict):
                v["frac_of_copy_bandwidth"] = round(v["GB/s"] * 1e9 / hbm, 4)
    kernels_alone = {"prompt_attention": {"puvolix": pp, "tarulix": tp, "minimax_m3": sp},
                     "single_token_attention": {"puvolix": pd, "tarulix": td, "minimax_m3": sd},
                     "recurrence_prompt": {"puvolix": gp, "guravik_delta_rule": dp, "tirizen_gla": lp},
                     "recurrence_single_tokens": {"puvolix": gd, "puvolix_batch_64": gd64, "guravik_delta_rule": dd, "tirizen_gla": ld},
                     "between_sublayers_prompt": bp, "between_sublayers_single_tokens": bd}
    for k_, v in kernels_alone.items():
        print(f"[bench] {k_}: {v}", file=sys.stderr, flush=True)
    first = next(iter(models.values()))["puvolix"] if models else {}
    return {"metric": f"Puvolix decode tokens/s (batch {args.batch}, {args.prompt_len}-token prompts) beside Tarulix and MiniMax-M3 at equal sizes",
            "value": first.get("decode_tok_s"), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": first.get("decode_ms"), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)", "design": "puvolix", "models": models,
            "kernels": kernels_alone, "peaks": {**pk, "source": pk_src}, "clocks": clocks.stop(),
            "gpu_launches": first.get("launches_per_decode_step", 0) * args.steps, "impl": "ours"}


def scan(tokens_per_req: int, reqs: int, inner: int, N: int, rank: int) -> dict:
    """``selective_scan`` alone (the float32 step projection, a library product, and the chain in time).  Bytes: the state read and written, and per token
    u (bfloat16), z, dt written and read, the output (bfloat16) and the projection row."""
    import torch
    import bench_kernels as bk
    from quanta_b200 import kernels as k
    dev = bk.DEV
    T = tokens_per_req * reqs
    u = torch.randn(T, inner, device=dev, dtype=torch.bfloat16)
    proj = torch.randn(T, rank + 2 * N, device=dev)
    z = torch.randn(T, inner, device=dev)
    w_dt = torch.randn(inner, rank, device=dev) / rank ** 0.5
    dt_b, D = torch.zeros(inner, device=dev), torch.ones(inner, device=dev)
    A = -torch.exp(torch.rand(inner, N, device=dev))
    layers = 1 if tokens_per_req > 1 else max(1, min(16, int(2e9 // (reqs * inner * N * 4))))
    states = [torch.zeros(reqs, inner, N, device=dev) for _ in range(layers)]
    out = torch.empty(T, inner, device=dev, dtype=torch.bfloat16)
    starts = torch.arange(0, T + 1, tokens_per_req, dtype=torch.int32, device=dev)
    slots = torch.arange(reqs, dtype=torch.int32, device=dev)

    def all_layers():
        for s in states:
            k.selective_scan(u, proj, z, torch.mm(proj[:, :rank], w_dt.t()), dt_b, A, D, s, out, starts, slots, rank, N)
    ms = (bk.timed_graph(all_layers, reps=1) if tokens_per_req == 1 else bk.timed(all_layers, n=5, warm=2)) / layers
    nbytes = 2 * reqs * inner * N * 4 + T * (inner * (2 + 4 + 8 + 2) + (rank + 2 * N) * 4) + inner * (rank + N + 2) * 4
    flops = T * inner * (2.0 * rank + 7.0 * N)
    return {"kernel": "selective_scan (steps + chain)", "requests": reqs, "tokens_per_request": tokens_per_req, "inner": inner,
            "state": N, "dt_rank": rank, "us": round(ms * 1e3, 2), "tokens/s": round(T / ms * 1e3, 1),
            "GB/s": round(nbytes / ms / 1e6, 1), "fp32 TFLOP/s": round(flops / ms / 1e9, 2)}


def run_tarulix(args) -> dict:
    import bench
    import bench_kernels as bk
    from quanta_b200.config import MiniMaxM3Config, TarulixConfig
    pk, pk_src = bench.peaks()
    clocks = bench.ClockSampler()
    clocks.start()
    models = {}
    for name, s in TARULIX_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        t0 = time.time()
        t = _model_numbers(TarulixConfig.from_dict(tarulix_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        m = _model_numbers(MiniMaxM3Config.from_dict(minimax_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        models[name] = {"sizes": s, "tarulix": t, "minimax_m3": m}
        print(f"[bench] {name}: tarulix {t}\n[bench] {name}: minimax_m3 {m} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    s = TARULIX_SIZES["w2048"]
    T, B = args.prompt_len, args.batch
    tensor, hbm = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    Hq, Hk, hd, W = s["attn_heads"], max(1, s["attn_heads"] // 4), s["dim"], s["window"]
    ctx = 4 * T                                         # single tokens deep into a context: the window is full
    wp = {kind: window_attn(T, 1, T, Hq, Hk, hd, W, kind, s["pool"]) for kind in ("biased", "pooled")}
    wd = {kind: window_attn(1, B, ctx, Hq, Hk, hd, W, kind, s["pool"]) for kind in ("biased", "pooled")}
    sp = bk.attn_span(T, 0, Hq, Hk, hd, 16)
    sd = bk.attn_decode(B, W, Hq, Hk, hd, 16)           # as many keys as the window holds
    for r in list(wp.values()) + [sp]:
        r["frac_of_tensor_peak"] = round(r["TFLOP/s"] * 1e12 / tensor, 4)
    for r in list(wd.values()) + [sd]:
        r["frac_of_copy_bandwidth"] = round(r["GB/s"] * 1e9 / hbm, 4)
    cp, cd = scan(T, 1, s["inner"], s["state"], s["dt_rank"]), scan(1, B, s["inner"], s["state"], s["dt_rank"])
    gp, gd = gla(T, 1, 32, 64, 64), gla(1, B, 32, 64, 64)
    for r in (cp, cd, gp, gd):
        r["frac_of_copy_bandwidth"] = round(r["GB/s"] * 1e9 / hbm, 4)
    kernels_alone = {"prompt_attention": {"tarulix": wp, "minimax_m3": sp}, "single_token_attention": {"tarulix": wd, "minimax_m3": sd},
                     "recurrence_prompt": {"tarulix": cp, "tirizen_gla": gp}, "recurrence_single_tokens": {"tarulix": cd, "tirizen_gla": gd}}
    for k_, v in kernels_alone.items():
        print(f"[bench] {k_}: {v}", file=sys.stderr, flush=True)
    first = next(iter(models.values()))["tarulix"] if models else {}
    return {"metric": f"Tarulix decode tokens/s (batch {args.batch}, {args.prompt_len}-token prompts) beside MiniMax-M3 at equal sizes",
            "value": first.get("decode_tok_s"), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": first.get("decode_ms"), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)", "design": "tarulix", "models": models,
            "kernels": kernels_alone, "peaks": {**pk, "source": pk_src}, "clocks": clocks.stop(),
            "gpu_launches": first.get("launches_per_decode_step", 0) * args.steps, "impl": "ours"}


def run(args) -> dict:
    if getattr(args, "design", "guravik") == "tirizen":
        return run_tirizen(args)
    if getattr(args, "design", "guravik") == "tarulix":
        return run_tarulix(args)
    if getattr(args, "design", "guravik") == "puvolix":
        return run_puvolix(args)
    import torch
    import bench
    import bench_kernels as bk
    from quanta_b200.config import GuravikConfig, MiniMaxM3Config
    pk, pk_src = bench.peaks()
    clocks = bench.ClockSampler()
    clocks.start()
    models = {}
    for name, s in SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        t0 = time.time()
        g = _model_numbers(GuravikConfig.from_dict(guravik_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        m = _model_numbers(MiniMaxM3Config.from_dict(minimax_raw(s)), args.prompt_len, args.batch, args.steps, args.warmup)
        models[name] = {"sizes": s, "guravik": g, "minimax_m3": m}
        print(f"[bench] {name}: guravik {g}\n[bench] {name}: minimax_m3 {m} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    s = SIZES["w2048"]
    C, R, Hh = s["kv_rank"], s["rot"], s["attn_heads"]
    T, B = args.prompt_len, args.batch
    tensor, hbm = pk["bf16_tflops"] * 1e12, pk["hbm_gbs"] * 1e9
    lp = latent_prefill(T, Hh, C, R)
    sp = bk.attn_span(T, 0, Hh, max(1, Hh // 4), 128, 16)
    ld = latent_decode(B, T, Hh, C, R)
    sd = bk.attn_decode(B, T, Hh, max(1, Hh // 4), 128, 16)
    dp = delta_rule(T, 1, s["delta_heads"], s["delta_dim"])
    dd = delta_rule(1, B, s["delta_heads"], s["delta_dim"])
    lp["frac_of_tensor_peak"] = round(lp["TFLOP/s"] * 1e12 / tensor, 4)
    sp["frac_of_tensor_peak"] = round(sp["TFLOP/s"] * 1e12 / tensor, 4)
    ld["frac_of_copy_bandwidth"] = round(ld["GB/s"] * 1e9 / hbm, 4)
    if "GB/s" in sd:
        sd["frac_of_copy_bandwidth"] = round(sd["GB/s"] * 1e9 / hbm, 4)
    dd["frac_of_copy_bandwidth"] = round(dd["GB/s"] * 1e9 / hbm, 4)
    kernels_alone = {"prompt_attention": {"guravik": lp, "minimax_m3": sp}, "single_token_attention": {"guravik": ld, "minimax_m3": sd},
                     "recurrence_prompt": dp, "recurrence_single_tokens": dd}
    for k_, v in kernels_alone.items():
        print(f"[bench] {k_}: {v}", file=sys.stderr, flush=True)
    first = next(iter(models.values()))["guravik"] if models else {}
    return {"metric": f"Guravik decode tokens/s (batch {args.batch}, {args.prompt_len}-token prompts) beside MiniMax-M3 at equal sizes",
            "value": first.get("decode_tok_s"), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": first.get("decode_ms"), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)", "design": "guravik", "models": models,
            "kernels": kernels_alone, "peaks": {**pk, "source": pk_src}, "clocks": clocks.stop(),
            "gpu_launches": first.get("launches_per_decode_step", 0) * args.steps, "impl": "ours"}


if __name__ == "__main__":
    # one kernel alone, one JSON line:  python bench_designs.py latent_prefill --tokens 1024
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["latent_prefill", "latent_decode", "delta_rule", "gla", "streams_norm", "window_prefill",
                                       "window_decode", "scan"])
    ap.add_argument("--kind", default="biased", choices=["biased", "pooled"])
    ap.add_argument("--window", type=int, default=1024)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--latent", type=int, default=256)
    ap.add_argument("--rot", type=int, default=64)
    ap.add_argument("--dim", type=int, default=64)
    a = ap.parse_args()
    if a.kernel == "latent_prefill":
        print(json.dumps(latent_prefill(a.tokens, a.heads, a.latent, a.rot)))
    elif a.kernel == "latent_decode":
        print(json.dumps(latent_decode(a.batch, a.tokens, a.heads, a.latent, a.rot)))
    elif a.kernel == "gla":
        print(json.dumps(gla(a.tokens, a.batch, a.heads, a.dim, a.dim)))
    elif a.kernel == "streams_norm":
        print(json.dumps(streams_norm(a.tokens, 3, 2048)))
    elif a.kernel == "window_prefill":
        print(json.dumps(window_attn(a.tokens, 1, a.tokens, a.heads, max(1, a.heads // 4), 128, a.window, a.kind)))
    elif a.kernel == "window_decode":
        print(json.dumps(window_attn(1, a.batch, a.tokens, a.heads, max(1, a.heads // 4), 128, a.window, a.kind)))
    elif a.kernel == "scan":
        print(json.dumps(scan(a.tokens, a.batch, 4096, 16, 128)))
    else:
        print(json.dumps(delta_rule(a.tokens, a.batch, a.heads, a.dim)))
