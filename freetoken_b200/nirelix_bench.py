"""Nirelix beside the Tonapel decoder at equal size: step throughput and kernel rooflines.

    python bench.py --design nirelix [--sizes w2048,w4096] [--steps K] [--warmup W]

For every size a four-layer Nirelix model (retention + dense, channel-decay delta rule + experts, latent
attention + experts, delta rule + dense; four residual streams; random weights) and the engine's closest
other model - a Tonapel decoder (window attention beside a state space, the gated delta rule, dense and
routed feed-forwards) of the same width, head counts, head size, layer count and vocabulary - run the
same workload through ``Engine.step`` (the method of :mod:`.design_bench`): one prompt of
``--prefill-tokens`` tokens, and decode steps at batch 8 and 1 on contexts of ``--context`` tokens
built by real prefill.

The second part times the design's own kernels beside the like kernel of the other model, each replayed
from a CUDA graph over inputs that are rotated so that no repetition finds them in L2, as a fraction of
the measured copy bandwidth: both new modes of the scan kernel beside the delta rule with one decay per
head (a prompt portion of 8,192 tokens, and a decode batch of 64 whose traffic is the states); the norm
over several residual streams beside ``rmsnorm`` and ``norm_add``; ``latent_store`` beside ``key_store``;
``rms_rows``; decode attention over rows of latent plus rotated part inside a window beside the same
kernel over a latent alone.  One JSON line.
"""

from __future__ import annotations

import json
import time
from typing import Any, Callable, Dict, List

from .design_bench import LAYERS, _timed, measure_model
from .tonapel_bench import tonapel_config

SIZES: Dict[str, Dict[str, int]] = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, ssd_heads=32, ssd_dim=64, state=128,
                  delta_heads=16, ff=8192, experts=8, top=2, vocab=32768, streams=4, q_rank=768, kv_rank=96, rot=32,
                  latent_dim=64, low_rank=64),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=1024, ssd_heads=64, ssd_dim=64, state=128,
                  delta_heads=32, ff=14336, experts=8, top=2, vocab=32768, streams=4, q_rank=1536, kv_rank=96, rot=32,
                  latent_dim=64, low_rank=128),
}
TAPS = 4


def nirelix_config(s: Dict[str, int]) -> Dict[str, Any]:
    d, H = s["dim"], s["delta_heads"]
    ret = {"heads": H, "dim": d, "vdim": d, "decay": [1.0 - 2.0 ** (-5 - (i % 8)) for i in range(H)],
           "rot": {"base": 1e4, "dims": d // 2}}
    delta = {"heads": H, "kv_heads": H, "dim": d, "vdim": d, "conv": TAPS, "low_rank": s["low_rank"]}
    lat = {"heads": s["heads"], "dim": s["latent_dim"], "rot_dim": s["rot"], "vdim": d, "q_rank": s["q_rank"],
           "kv_rank": s["kv_rank"], "scale": (s["latent_dim"] + s["rot"]) ** -0.5, "mask": {"size": s["window"]},
           "rot": {"base": 1e4, "dims": s["rot"]}}
    inter = max(128, (s["ff"] // 3) // 128 * 128)
    dense = {"kind": "dense", "ff": s["ff"] * 2 // 3 // 128 * 128, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": inter},
           "router": {"experts": s["experts"], "top": s["top"], "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
    return {"architecture": "Nirelix", "vocab": s["vocab"], "width": s["width"], "streams": s["streams"],
            "norm": {"eps": 1e-6},
            "layers": [{"type": "retention", "mixer": ret, "mlp": dense}, {"type": "channel_delta", "mixer": delta, "mlp": moe},
                       {"type": "latent_attention", "mixer": lat, "mlp": moe},
                       {"type": "channel_delta", "mixer": delta, "mlp": dense}]}


def kernel_pairs(s: Dict[str, int], peaks: Dict[str, Any], reps: int = 10) -> Dict[str, Any]:
    import torch

    from .csrc import ops
    from .parts.base import Workspace
    from .parts.position import rotary_table

    dev, bf = "cuda:0", torch.bfloat16
    hbm = peaks["hbm_gbs"] * 1e9
    W, d, P, S_ = s["width"], s["dim"], 64, s["streams"]
    out: Dict[str, Any] = {}

    def rotate(make: Callable[[], Any], nbytes: int, most: int = 16) -> List[Any]:
        return [make() for _ in range(min(most, max(2, -(-(256 << 20) // max(1, nbytes)))))]

    def run(name: str, launch: Callable[[int], None], sets: int, nbytes: float) -> None:
        for i in range(min(sets, 3)):
            launch(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(sets):
                launch(i)
        graph.replay()
        ms = _timed(graph.replay, reps) / sets
        out[name] = {"us": round(ms * 1e3, 2), "gbs": round(nbytes / (ms / 1e3) / 1e9, 1),
                     "frac_of_measured_copy_peak": round(nbytes / (ms / 1e3) / hbm, 3)}

    def meta(lens):
        q = [0]
        for n in lens:
            q.append(q[-1] + n)
        seg = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(lens)]).to(dev)
        return (seg, torch.arange(len(lens), dtype=torch.int32, device=dev),
                torch.tensor(q, dtype=torch.int32, device=dev))

    Hd = s["delta_heads"]
    Cd = 3 * Hd * d
    cos_sin = rotary_table(d // 2, 1e4, dev, 8192, exact_angles=True)
    for label, lens in (("one prompt portion of 8,192 tokens", [8192]), ("decode batch of 64", [1] * 64)):
        T, S = sum(lens), len(lens)
        seg, slot, q = meta(lens)
        pos0 = torch.full((S,), 0 if S == 1 else 2047, dtype=torch.int32, device=dev)
        state_b = Hd * d * d * 4
        qs = rotate(lambda: torch.randn(T, Cd, device=dev, dtype=bf), T * Cd * 2 + S * state_b)
        states = [torch.zeros(S, Hd * d * d, device=dev) for _ in qs]
        gates = torch.randn(T, 2 * Hd, device=dev, dtype=bf)
        decay32 = torch.randn(T, Hd * d, device=dev)
        small = [torch.zeros(Hd, device=dev), torch.zeros(Hd, device=dev), torch.zeros(Hd * d, device=dev),
                 torch.full((Hd,), 0.99, device=dev)]
        o = torch.empty(T, Hd * d, device=dev)
        base = T * Cd * 2 + T * Hd * d * 4 + 2 * S * state_b
        run(f"delta_scan (one decay a head), {label}",
            lambda i: ops.delta_scan(qs[i], gates[:, :Hd], gates[:, Hd:], small[0], small[1], states[i], o, slot, q,
                                     Hd, Hd, d, d, 1e-6, d ** -0.5), len(qs), nbytes=base)
        run(f"channel_delta_scan (a decay a key channel), {label}",
            lambda i: ops.channel_delta_scan(qs[i], gates[:, :Hd], decay32, small[2], small[1], states[i], o, slot, q,
                                             Hd, Hd, d, d, 1e-6, d ** -0.5), len(qs), nbytes=base + T * Hd * d * 4)
        run(f"retention_scan (rotation inside), {label}",
            lambda i: ops.retention_scan(qs[i], small[3], cos_sin, pos0, states[i], o, slot, q, Hd, d, d, d ** -0.5),
            len(qs), nbytes=base)
        del qs, states
        # ---- the norm over several streams beside the norms over one -------------------------------
        branches = rotate(lambda: torch.randn(T, W, device=dev, dtype=bf), T * W * (2 + 8 * S_ + 2), most=8)
        streams = torch.zeros(T, S_, W, device=dev)
        res = torch.zeros(T, W, device=dev)
        w1, b1 = torch.ones(W, device=dev), torch.zeros(W, device=dev)
        mix = torch.eye(S_, device=dev)
        ones = torch.ones(S_, device=dev)
        nout = torch.empty(T, W, device=dev, dtype=bf)
        run(f"hyper_norm ({S_} streams: join, read, layer norm), {label}",
            lambda i: ops.hyper_norm(streams, branches[i], mix, ones, ones, w1, b1, 1e-6, True, nout), len(branches),
            nbytes=T * W * (2 + 8 * S_ + 2))
        one = torch.zeros(T, 1, W, device=dev)
        run(f"hyper_norm (1 stream), {label}",
            lambda i: ops.hyper_norm(one, branches[i], mix[:1, :1].contiguous(), ones[:1], ones[:1], w1, b1, 1e-6, True,
                                     nout), len(branches), nbytes=T * W * (2 + 8 + 2))
        run(f"rmsnorm (residual add + norm), {label}",
            lambda i: ops.rmsnorm(branches[i], res, w1, nout, 1e-6, False), len(branches), nbytes=T * W * (2 + 8 + 2))
        del branches

    # ---- latent rows -> cache and query tails, beside the latent store without rotation -------------
    T = 8192
    H, R, rot, dq = s["heads"], s["kv_rank"], s["rot"], s["latent_dim"]
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seg0 = torch.zeros(T, dtype=torch.int32, device=dev)
    table = torch.arange(1, T // P + 1, dtype=torch.int32, device=dev).view(1, -1)
    downs = rotate(lambda: torch.randn(T, R + rot, device=dev, dtype=bf), T * (R + rot) * 2 * 4)
    qrows = torch.randn(T, H * (dq + rot), device=dev, dtype=bf)
    q_abs = torch.empty(T, H, R + rot, device=dev, dtype=bf)
    pages = torch.zeros(T // P + 1, 1, P, R + rot, device=dev, dtype=bf)
    nw = torch.ones(R, device=dev)
    cs = rotary_table(rot, 1e4, dev, T, exact_angles=True)
    run("latent_store (norm, rotation, cache row, query tails), 8,192 tokens",
        lambda i: ops.latent_store(downs[i], qrows, q_abs, pages, nw, cs, pos, seg0, table, heads=H, q_dim=dq, rank=R,
                                   rot=rot, interleaved=True, eps=1e-6), len(downs),
        nbytes=T * ((R + rot) * 2 * 2 + H * rot * 2 * 2))
    pages1 = torch.zeros(T // P + 1, 1, P, R + rot, device=dev, dtype=bf)
    nw1 = torch.ones(R + rot, device=dev)
    run("key_store (latent: norm + cache row), 8,192 tokens",
        lambda i: ops.key_store(downs[i], None, pages1, nw1, pos, seg0, table, q_off=0, k_off=0, num_heads=H, q_dim=dq,
                                num_kv_heads=1, k_dim=R + rot, eps=1e-6), len(downs), nbytes=T * (R + rot) * 2 * 2)
    qr = s["q_rank"]
    wides = rotate(lambda: torch.randn(T, qr, device=dev, dtype=bf), T * qr * 4, most=8)
    cq = torch.empty(T, qr, device=dev, dtype=bf)
    nq = torch.ones(qr, device=dev)
    run("rms_rows (query latent), 8,192 tokens", lambda i: ops.rms_rows(wides[i], nq, cq, 1e-6), len(wides),
        nbytes=T * qr * 4)
    del downs, wides

    # ---- decode attention, 64 requests at position 2,047, one shared row of rank + rot values -------
    B, ctx, dd = 64, 2048, R + rot
    ws = Workspace(dev)
    per_req = ctx // P
    n_pages = B * per_req
    dpos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    dseg = torch.arange(B, dtype=torch.int32, device=dev)
    dtable = torch.arange(1, n_pages + 1, dtype=torch.int32, device=dev).view(B, per_req)
    planes = rotate(lambda: torch.randn(n_pages + 1, 1, P, dd, device=dev, dtype=bf), (n_pages + 1) * P * dd * 2, most=3)
    both = [p.unsqueeze(0).expand(2, *p.shape) for p in planes]
    qd = torch.randn(B, H * dd, device=dev, dtype=bf)
    od = torch.empty_like(qd)
    if ops.attn_decode_takes(qd, dd):
        for name, window in ((f"attn_decode over latent rows inside a window of {s['window']}", s["window"]),
                             ("attn_decode over latent rows, all 2,048 keys", None)):
            keys = window or ctx
            run(name, lambda i, w=window: ops.attn_decode(qd, od, both[i], None, B, dpos, dseg, dtable, H, 1, dd,
                                                          dd ** -0.5, w, ctx, ws), len(both), nbytes=B * keys * dd * 2)
    # rows that are no size of the tensor-core kernels (384 + 64 values) go to the generic kernel
    dd2 = 448
    planes2 = rotate(lambda: torch.randn(n_pages + 1, 1, P, dd2, device=dev, dtype=bf), (n_pages + 1) * P * dd2 * 2, most=2)
    both2 = [p.unsqueeze(0).expand(2, *p.shape) for p in planes2]
    q2 = torch.randn(B, H * dd2, device=dev, dtype=bf)
    o2 = torch.empty_like(q2)
    run(f"attention over latent rows of {dd2} values (generic kernel), window {s['window']}",
        lambda i: ops.attn_paged_simt(q2, o2, both2[i], dpos, dseg, dtable, H, 1, dd2, dd2 ** -0.5, s["window"]),
        len(both2), nbytes=B * s["window"] * dd2 * 2)
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
            sizes[n] = {"shape": s, "nirelix": measure_model(nirelix_config(s), a),
                        "tonapel_equal_size": measure_model(tonapel_config(s), a)}
        kernels = kernel_pairs(SIZES[names[0]], peaks)
    torch.cuda.synchronize()
    line = {"bench": "design", "design": "Nirelix", "beside": "Tonapel decoder at equal size",
            "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids", "layers": LAYERS,
            "context": a.context, "steps": a.steps, "warmup": max(3, a.warmup), "sizes": sizes,
            "kernels_at": names[0], "kernels": kernels,
            "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"], "source": peaks["source"]},
            "clocks": clocks.summary(), "wall_s": round(time.time() - t0, 1)}
    print(json.dumps(line))
    return 0
