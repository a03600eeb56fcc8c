"""Mezapel beside the MiniMax-M3 decoder at equal size: step throughput and kernel rooflines.

    python bench.py --design mezapel [--sizes w2048,w4096] [--steps K] [--warmup W]

For every size a four-layer Mezapel model (chunked attention with a sink of score 0 and a gate per head,
twice the windowed attention behind short convolutions with capped scores, a learned sink and a gate per
value, chunked attention again; four residual streams joined by hyper-connections; an embedding with a
hashed second table; dense gated feed-forwards; random weights) and the engine's closest other model - the
MiniMax-M3 decoder, whose mixer is the same grouped-query attention part without these options, at the
same width, head counts, head size, layer count and vocabulary, with experts sized to the same active
feed-forward weights - run the same workload through ``Engine.step`` (the method of :mod:`.design_bench`):
one prompt of ``--prefill-tokens`` tokens, and decode steps at batch 8 and 1 on contexts of ``--context``
tokens built by real prefill.

The second part times the design's own kernels beside the like kernel of the other model, each replayed
from a CUDA graph over inputs that are rotated so that no repetition finds them in L2, as a fraction of
the measured copy bandwidth (prompt attention: of the measured bfloat16 rate, counting the query-key
pairs the mask leaves): the embedding with the hashed table beside ``embed_gather``; the convolution
without activation beside ``conv_silu``; decode and prompt attention with chunks and a sink, and with a
window, a cap and a learned sink, beside the same kernels with a plain window; both gates.  One JSON line.
"""

from __future__ import annotations

import json
import time
from typing import Any, Callable, Dict, List

from .design_bench import LAYERS, _timed, measure_model, minimax_config

SIZES: Dict[str, Dict[str, int]] = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, chunk=1024, ff=8192, vocab=32768,
                  streams=4, buckets=65521),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=1024, chunk=1024, ff=14336, vocab=32768,
                  streams=4, buckets=65521),
}
TAPS = 4


def mezapel_config(s: Dict[str, int]) -> Dict[str, Any]:
    d = s["dim"]
    chunked = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5,
               "mask": {"size": s["chunk"]},
               "rot": {"base": 10000.0, "dims": d // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    windowed = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5,
                "mask": {"size": s["window"]}, "conv": TAPS, "softcap": 50.0,
                "rot": {"base": 500000.0, "dims": d, "scaling": {"factor": 16.0, "original": 8192, "low": 1.0, "high": 8.0}}}
    mlp = {"kind": "dense", "ff": s["ff"] * 2 // 3 // 128 * 128}
    return {"architecture": "Mezapel", "vocab": s["vocab"], "width": s["width"], "streams": s["streams"],
            "norm": {"eps": 1e-6},
            "embedding": {"scale": float(s["width"]) ** 0.5, "bigram": {"buckets": s["buckets"], "mul_prev": 36313, "mul_cur": 27191}},
            "layers": [{"type": "attention", "mixer": chunked, "mlp": mlp}, {"type": "attention_2", "mixer": windowed, "mlp": mlp},
                       {"type": "attention_2", "mixer": windowed, "mlp": mlp}, {"type": "attention", "mixer": chunked, "mlp": mlp}]}


def kernel_pairs(s: Dict[str, int], peaks: Dict[str, Any], reps: int = 10) -> Dict[str, Any]:
    import torch

    from .csrc import ops
    from .parts.base import Workspace

    dev, bf = "cuda:0", torch.bfloat16
    hbm, tflops = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    W, d, P, S_ = s["width"], s["dim"], 64, s["streams"]
    H, G = s["heads"], s["kv_heads"]
    out: Dict[str, Any] = {}

    def rotate(make: Callable[[], Any], nbytes: int, most: int = 16) -> List[Any]:
        return [make() for _ in range(min(most, max(2, -(-(256 << 20) // max(1, nbytes)))))]

    def run(name: str, launch: Callable[[int], None], sets: int, nbytes: float = 0.0, flops: float = 0.0) -> None:
        for i in range(min(sets, 3)):
            launch(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(sets):
                launch(i)
        graph.replay()
        ms = _timed(graph.replay, reps) / sets
        out[name] = {"us": round(ms * 1e3, 2)}
        if nbytes:
            out[name].update(gbs=round(nbytes / (ms / 1e3) / 1e9, 1),
                             frac_of_measured_copy_peak=round(nbytes / (ms / 1e3) / hbm, 3))
        if flops:
            out[name].update(tflops=round(flops / (ms / 1e3) / 1e12, 1),
                             frac_of_measured_bf16_peak=round(flops / (ms / 1e3) / tflops, 3))

    # ---- embedding: token row times a factor plus the hashed row, into every stream -------------------
    T = 8192
    V, B_ = s["vocab"], s["buckets"]
    emb = torch.randn(V, W, device=dev, dtype=bf)
    pair = torch.randn(B_ + 1, W, device=dev, dtype=bf)
    ids = [torch.randint(0, V, (T,), dtype=torch.int32, device=dev) for _ in range(4)]
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seg0 = torch.zeros(T, dtype=torch.int32, device=dev)
    slot0 = torch.zeros(1, dtype=torch.int32, device=dev)
    q0 = torch.tensor([0, T], dtype=torch.int32, device=dev)
    last = torch.zeros(2, 1, dtype=torch.int32, device=dev)
    res = torch.empty(T, S_, W, device=dev)
    res1 = torch.empty(T, 1, W, device=dev)
    run(f"embed_pair (scale, hashed second table, {S_} streams), 8,192 tokens",
        lambda i: ops.embed_pair(ids[i], pos, seg0, slot0, q0, emb, pair, last, res, 3.0, B_, 36313, 27191), 4,
        nbytes=T * W * (2 * 2 + 4 * S_))
    run("embed_pair (1 stream), 8,192 tokens",
        lambda i: ops.embed_pair(ids[i], pos, seg0, slot0, q0, emb, pair, last, res1, 3.0, B_, 36313, 27191), 4,
        nbytes=T * W * (2 * 2 + 4))
    run("embed_gather (1 stream), 8,192 tokens", lambda i: ops.embed_gather(ids[i], emb, res1), 4, nbytes=T * W * (2 + 4))
    del emb, pair, res, res1

    # ---- the convolution behind q, k and v, without and with activation ----------------------------------
    C = (H + 2 * G) * d
    for label, lens in (("one prompt portion of 8,192 tokens", [8192]), ("decode batch of 64", [1] * 64)):
        Tn, S = sum(lens), len(lens)
        q = [0]
        for n in lens:
            q.append(q[-1] + n)
        seg = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(dev)
        slot = torch.arange(S, dtype=torch.int32, device=dev)
        qs = torch.tensor(q, dtype=torch.int32, device=dev)
        xs = rotate(lambda: torch.randn(Tn, C + H * d, device=dev, dtype=bf), Tn * C * 4, most=8)
        states = [torch.zeros(S, (TAPS - 1) * C, device=dev) for _ in xs]
        cw = torch.randn(C, TAPS, device=dev)
        cout = torch.empty(Tn, C, device=dev, dtype=bf)
        nbytes = 2 * Tn * C * 2 + 2 * S * (TAPS - 1) * C * 4
        run(f"conv (no activation) over q, k, v, {label}",
            lambda i: ops.conv_silu(xs[i][:, :C], cout, cw, None, states[i], seg, slot, qs, activation=False), len(xs), nbytes=nbytes)
        run(f"conv_silu, {label}", lambda i: ops.conv_silu(xs[i][:, :C], cout, cw, None, states[i], seg, slot, qs), len(xs),
            nbytes=nbytes)
        # ---- gates: one per head, one per value -------------------------------------------------------
        o = torch.randn(Tn, H * d, device=dev, dtype=bf)
        run(f"gate_heads (a gate a head), {label}", lambda i: ops.gate_heads(o, xs[i][:, C:C + H], H, d), len(xs),
            nbytes=Tn * H * d * 4)
        run(f"gate_heads (a gate a value), {label}", lambda i: ops.gate_heads(o, xs[i][:, C:], H * d, 1), len(xs),
            nbytes=Tn * H * d * 6)
        del xs, states

    # ---- decode attention, 64 requests at position 2,047 ------------------------------------------------
    Bn, ctx = 64, 2048
    ws = Workspace(dev)
    per_req = ctx // P
    n_pages = Bn * per_req
    dpos = torch.full((Bn,), ctx - 1, dtype=torch.int32, device=dev)
    dseg = torch.arange(Bn, dtype=torch.int32, device=dev)
    dtable = torch.arange(1, n_pages + 1, dtype=torch.int32, device=dev).view(Bn, per_req)
    caches = rotate(lambda: torch.randn(2, n_pages + 1, G, P, d, device=dev, dtype=bf), 2 * (n_pages + 1) * G * P * d * 2, most=3)
    qd = torch.randn(Bn, H * d, device=dev, dtype=bf)
    od = torch.empty_like(qd)
    sink = torch.randn(H, device=dev)
    keys = s["window"]
    variants = (("chunks of %d, a sink of score 0" % s["chunk"], None, ops.ScoreOptions(chunk=s["chunk"], sink_value=0.0)),
                ("a window of %d, capped scores, a learned sink" % s["window"], s["window"], ops.ScoreOptions(softcap=50.0, sink=sink)),
                ("a window of %d, plain" % s["window"], s["window"], None))
    for label, window, options in variants:
        run(f"attn_decode, 64 x 2,048 keys, {label}",
            lambda i, w=window, o_=options: ops.attn_decode(qd, od, caches[i], None, Bn, dpos, dseg, dtable, H, G, d, d ** -0.5, w,
                                                            ctx, ws, options=o_), len(caches), nbytes=Bn * keys * G * d * 2 * 2)
    del caches

    # ---- prompt attention, one portion of 8,192 tokens: the tcgen05 kernel, and the tiled mma.sync kernel
    # that small steps take ---------------------------------------------------------------------------
    T = 8192
    pages = T // P
    kv = torch.randn(2, pages + 1, G, P, d, device=dev, dtype=bf)
    table = torch.arange(1, pages + 1, dtype=torch.int32, device=dev).view(1, pages)
    qp = torch.randn(T, H * d, device=dev, dtype=bf)
    op = torch.empty_like(qp)
    tile_seg = torch.zeros(T // 64, dtype=torch.int32, device=dev)
    tile_q0 = torch.arange(0, T, 64, dtype=torch.int32, device=dev)
    starts = torch.tensor([0, T], dtype=torch.int32, device=dev)
    p0 = torch.zeros(1, dtype=torch.int32, device=dev)
    w = s["window"]
    pairs_window = sum(min(i + 1, w) for i in range(T))
    pairs_chunk = sum(i % s["chunk"] + 1 for i in range(T))
    for label, window, options, pairs in (
            ("chunks of %d, a sink of score 0" % s["chunk"], None, ops.ScoreOptions(chunk=s["chunk"], sink_value=0.0), pairs_chunk),
            ("a window of %d, capped scores, a learned sink" % w, w, ops.ScoreOptions(softcap=50.0, sink=sink), pairs_window),
            ("a window of %d, a learned sink" % w, w, ops.ScoreOptions(sink=sink), pairs_window),
            ("a window of %d, plain" % w, w, None, pairs_window)):
        run(f"attn_prefill (mma.sync), 8,192 tokens, {label}",
            lambda i, w_=window, o_=options: ops.attn_prefill(qp, op, kv, tile_seg, tile_q0, starts, p0, table, H, G, d, d ** -0.5,
                                                              w_, options=o_), 2, flops=4.0 * pairs * H * d)
        run(f"attn_prefill_tc (tcgen05), 8,192 tokens, {label}",
            lambda i, w_=window, o_=options: ops.attn_prefill_tc(qp, op, kv, tile_seg, tile_q0, starts, p0, table, H, G, d,
                                                                 d ** -0.5, w_, options=o_), 2, flops=4.0 * pairs * H * d)
    run("attn_prefill_tc (tcgen05), 8,192 tokens, all keys, plain",
        lambda i: ops.attn_prefill_tc(qp, op, kv, tile_seg, tile_q0, starts, p0, table, H, G, d, d ** -0.5), 2,
        flops=4.0 * (T * (T + 1) // 2) * H * d)
    return out


def main(a) -> int:
    import torch

    from .benchmark import ClockSampler, load_peaks

    peaks = load_peaks()
    names = [n for n in a.sizes.split(",") if n.strip()]
    for n in names:
        if n not in SIZES:
            print(f"unknown size '{n}' (known: {', '.join(SIZES)})")
            return 2
    t0 = time.time()
    sizes: Dict[str, Any] = {}
    with ClockSampler() as clocks:
        for n in names:
            s = SIZES[n]
            room = a.context + a.steps + a.warmup + 16 + 3 * 64
            sizes[n] = {"shape": s, "mezapel": measure_model(mezapel_config(s), a),
                        "minimax_m3_equal_size": measure_model(minimax_config({**s, "rank": 0}, room), a)}
        kernels = kernel_pairs(SIZES[names[0]], peaks)
    torch.cuda.synchronize()
    line = {"bench": "design", "design": "Mezapel", "beside": "MiniMax-M3 decoder at equal size",
            "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids", "layers": LAYERS,
            "context": a.context, "steps": a.steps, "warmup": max(3, a.warmup), "sizes": sizes,
            "kernels_at": names[0], "kernels": kernels,
            "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": peaks["source"]},
            "clocks": clocks.summary(), "wall_s": round(time.time() - t0, 1)}
    print(json.dumps(line))
    return 0
