"""Mezapel in the engine against the plain implementation: every new kernel alone, every mechanism
alone in a one-layer model, whole prompts against decoding, portions down to two tokens, mixed
batches with pages and state slots used again, the edge of a chunk and of a window and a key far
back made decisive on purpose, the first tokens, long decoding, four configurations that differ in
every size, greedy generation through the scheduler, the trace replay tool."""

import math

import pytest
import torch

import mezapel_tiny as mz
import plain_mezapel as plain
import replay_driver as rd

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 150, 66, 260, 21], "C": [2, 35, 77, 5], "D": [1, 40, 13, 26, 2]}
CUTS = {"whole": rd.whole, "decode_tail": rd.decode_tail, "portions": rd.portions, "mixed": rd.mixed}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DEV = "cuda"


def requests_of(which):
    vocab = mz.MZ[which]["vocab"]
    return {f"r{i}": mz.tokens(30 * i + ord(which), n, vocab) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {which: mz.write_tiny(str(tmp_path_factory.mktemp(f"mz{which}")), which) for which in mz.MZ}


def run_and_compare(folder, config, state, reqs, schedule, dtype, page, what, tol=None, poison=True, want=None):
    engine = mz.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=poison)
    got = rd.run_engine(engine, reqs, schedule)
    want = want or {rid: plain.forward(config, state, toks) for rid, toks in reqs.items()}
    mz.compare(got, want, tol or mz.TOL[dtype], f"{what} [{dtype}]")
    assert engine.cache.free_pages() == engine.cache.total_pages()
    return got


def close(got, want, dtype, what=""):
    tol = 2e-5 if dtype == "float32" else 2e-2
    g, w = got.double().cpu(), want.double()
    assert torch.allclose(g, w, atol=tol * max(1.0, float(w.abs().max())), rtol=tol), (what, float((g - w).abs().max()))


# ------------------------------------------------------------------ kernels, each alone
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,copies,buckets,mul_prev,mul_cur", [(40, 1, 7, 5, 3), (70, 3, 1, 2, 9), (256, 4, 1019, 100003, 99991)])
def test_embed_pair(dtype, H, copies, buckets, mul_prev, mul_cur):
    """Three requests in slots 2, 0 and 3 over two steps: portions that start a sequence, that go on
    (the token before comes from the slot), single tokens; multipliers whose products pass 2^31."""
    from freetoken_b200.csrc import ops
    vocab = 50000 if buckets > 1000 else 33
    torch.manual_seed(H)
    table = torch.randn(vocab, H).to(DTYPES[dtype])
    pair = torch.randn(buckets + 1, H).to(DTYPES[dtype])
    seqs = {2: mz.tokens(1, 9, vocab), 0: mz.tokens(2, 4, vocab), 3: mz.tokens(3, 6, vocab)}
    state = torch.full((5, 3), -1, dtype=torch.int32, device=DEV)[:, :1]           # rows lie 3 apart
    steps = [[(2, 0, 5), (0, 0, 1), (3, 0, 2)], [(0, 1, 3), (2, 5, 4), (3, 2, 1)], [(3, 3, 3)]]
    big = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    for step in steps:
        ids, pos, seg, slot, q0 = [], [], [], [], [0]
        for i, (s, first, n) in enumerate(step):
            ids += seqs[s][first:first + n]
            pos += list(range(first, first + n))
            seg += [i] * n
            slot.append(s)
            q0.append(q0[-1] + n)
        dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
        shape = (len(ids), copies, H) if copies > 1 else (len(ids), H)
        residual = torch.full(shape, float("nan"), device=DEV)
        ops.embed_pair(dev(ids), dev(pos), dev(seg), dev(slot), dev(q0), table.to(DEV), pair.to(DEV), state, residual,
                       1.75, buckets, mul_prev, mul_cur)
        row = 0
        for s, first, n in step:
            rows = plain.bigram_rows(seqs[s][:first + n], big)[first:]
            want = table[seqs[s][first:first + n]].double() * 1.75 + pair[rows].double()
            for c in range(copies):
                got = residual[row:row + n, c] if copies > 1 else residual[row:row + n]
                assert torch.allclose(got.double().cpu(), want, rtol=1e-6, atol=1e-6), (s, first, c)
            assert int(state[s, 0]) == seqs[s][first + n - 1]
            row += n
    # without a second table: only the factor
    residual = torch.empty(4, H, device=DEV)
    ids = torch.tensor([1, 0, 5, 1], dtype=torch.int32, device=DEV)
    ops.embed_pair(ids, None, None, None, None, table.to(DEV), None, None, residual, -0.5)
    assert torch.allclose(residual.cpu(), table[ids.cpu().long()].float() * -0.5)


def paged_case(dtype, nq, nkv, d, P, lens, seed=0):
    """Segments given as (pos0, n); K/V for positions < pos0 + n live in shuffled pages."""
    S = len(lens)
    width = max(-(-(p + n) // P) for p, n in lens)
    pages = S * width + 1
    g = torch.Generator().manual_seed(seed)
    table = (torch.randperm(pages - 1, generator=g)[: S * width] + 1).to(torch.int32).view(S, width)
    kv = torch.randn(2, pages, nkv, P, d, generator=g).to(DTYPES[dtype])
    T = sum(n for _, n in lens)
    q = (torch.randn(T, nq * d, generator=g) * 1.5).to(DTYPES[dtype])
    pos, seg = [], []
    for s, (p0, n) in enumerate(lens):
        pos += list(range(p0, p0 + n))
        seg += [s] * n
    return q, kv, pos, seg, table


def attention_reference(q, kv, pos, seg, table, nq, nkv, d, P, scale, window, chunk, cap, sinks):
    """Row by row with the plain implementation's softmax: ``sinks`` is None or a score per head."""
    T = q.shape[0]
    out = torch.zeros(T, nq, d, dtype=torch.float64)
    qf, kvf = q.double().view(T, nq, d), kv.double()
    for t in range(T):
        p, s = pos[t], seg[t]
        keys = torch.stack([kvf[0, int(table[s, j // P]), :, j % P] for j in range(p + 1)])       # [p + 1, nkv, d]
        vals = torch.stack([kvf[1, int(table[s, j // P]), :, j % P] for j in range(p + 1)])
        if chunk:
            visible = lambda a, b: b <= p and p // chunk == b // chunk
        else:
            visible = lambda a, b: 0 <= p - b < (window or p + 1)
        for h in range(nq):
            g = h // (nq // nkv)
            scores = (keys[:, g] @ qf[t, h]) * scale
            if cap:
                scores = cap * torch.tanh(scores / cap)
            sink = -math.inf if sinks is None else float(sinks[h])
            w = plain.masked_softmax_with_sink(scores[None, :], visible, sink)[0]
            out[t, h] = w @ vals[:, g]
    return out.view(T, nq * d)


OPTION_CASES = [
    # nq, nkv, d, P, segments (pos0, n), window, chunk, cap, sink (None | "zero" | "learned")
    (4, 2, 16, 4, [(0, 9), (21, 3), (7, 1)], None, 5, 0.0, "zero"),
    (6, 1, 24, 8, [(0, 20), (37, 1), (16, 1)], 6, None, 3.0, "learned"),
    (3, 3, 40, 16, [(31, 2), (64, 1), (63, 1)], None, 32, 2.0, None),
    (4, 2, 64, 64, [(100, 70), (255, 1), (256, 1), (0, 1)], None, 128, 0.0, "zero"),        # chunk = two pages
    (8, 2, 128, 64, [(60, 10), (300, 1), (127, 2)], 100, None, 8.0, "learned"),
    (5, 5, 32, 8, [(0, 66), (130, 1)], None, 1, 0.0, "zero"),                               # every key alone with the sink
    (16, 1, 64, 16, [(500, 1), (40, 65)], None, 200, 4.0, "learned"),
    (4, 4, 128, 128, [(1000, 3), (0, 2), (1279, 1), (1280, 1)], None, 640, 0.0, "learned"),
    (2, 1, 80, 32, [(90, 45)], 33, None, 12.0, "learned"),                                   # a head size only the generic kernel takes
    (4, 2, 128, 64, [(0, 300), (700, 130), (5, 1)], 100, None, 0.0, "learned"),             # a window that starts inside key tiles
    (3, 1, 64, 64, [(30, 260), (0, 2)], None, 96, 6.0, "zero"),                             # chunks across tiles; three heads a key head
    (2, 2, 128, 128, [(250, 200)], 64, None, 0.0, None),                                     # a window of one tile, nothing else
    (4, 1, 64, 64, [(1000, 150), (64, 64)], None, 512, 25.0, "learned"),
    (2, 1, 64, 64, [(0, 130), (200, 1)], 1, None, 0.0, "learned"),                           # a window of one: only the sink beside the key itself
    (2, 2, 128, 64, [(60, 70), (129, 1)], None, 1, 5.0, "zero"),
    (24, 1, 64, 64, [(300, 1), (10, 66)], 150, None, 0.0, "learned"),                        # 24 heads a key head: two head tiles in decoding
]


def _options(sink, nq, chunk, cap, seed=3):
    from freetoken_b200.csrc import ops
    g = torch.Generator().manual_seed(seed)
    learned = (torch.randn(nq, generator=g) * 2.0 + 4.0) if sink == "learned" else None
    sinks = learned if sink == "learned" else (torch.zeros(nq) if sink == "zero" else None)
    opts = ops.ScoreOptions(chunk or 0, cap, 0.0 if sink == "zero" else None, learned.to(DEV) if learned is not None else None)
    return opts, sinks


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("nq,nkv,d,P,lens,window,chunk,cap,sink", OPTION_CASES)
def test_attention_options_generic_kernel(dtype, nq, nkv, d, P, lens, window, chunk, cap, sink):
    from freetoken_b200.csrc import ops
    q, kv, pos, seg, table = paged_case(dtype, nq, nkv, d, P, lens)
    opts, sinks = _options(sink, nq, chunk, cap)
    dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q, device=DEV)
    scale = 1.3 * d ** -0.5
    ops.attn_paged_simt(q.to(DEV), out, kv.to(DEV), dev(pos), dev(seg), table.to(DEV), nq, nkv, d, scale, window, options=opts)
    want = attention_reference(q, kv, pos, seg, table, nq, nkv, d, P, scale, window, chunk, cap, sinks)
    close(out, want, dtype)
    if sinks is not None:
        # the sink is not a detail: without it the same rows come out visibly different
        bare = attention_reference(q, kv, pos, seg, table, nq, nkv, d, P, scale, window, chunk, cap, None)
        assert float((bare - want).abs().max()) > 0.05


@pytest.mark.parametrize("nq,nkv,d,P,lens,window,chunk,cap,sink", [c for c in OPTION_CASES if c[2] in (32, 64, 128)])
def test_attention_options_tensor_core_kernels(nq, nkv, d, P, lens, window, chunk, cap, sink):
    """Single-token segments through the split-KV decode kernels (cp.async and TMA-fed, splits merged by
    a cluster and by the merge kernel, one split and many), longer ones through the tiled prefill kernel."""
    from freetoken_b200.csrc import ops
    from freetoken_b200.parts.base import Workspace
    q, kv, pos, seg, table = paged_case("bfloat16", nq, nkv, d, P, lens)
    opts, sinks = _options(sink, nq, chunk, cap)
    dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    scale = 1.3 * d ** -0.5
    want = attention_reference(q, kv, pos, seg, table, nq, nkv, d, P, scale, window, chunk, cap, sinks)
    starts = [0]
    for _, n in lens:
        starts.append(starts[-1] + n)
    qd, kvd, posd, segd, tabled = q.to(DEV), kv.to(DEV), dev(pos), dev(seg), table.to(DEV)
    single = [starts[i] for i, (_, n) in enumerate(lens) if n == 1]
    tiles = [(s, q0) for s, (_, n) in enumerate(lens) if n > 1 for q0 in range(0, n, 64)]
    many = [starts[i] + r for i, (_, n) in enumerate(lens) if n > 1 for r in range(n)]
    if tiles:
        out = torch.zeros_like(qd)
        ops.attn_prefill(qd, out, kvd, dev([t[0] for t in tiles]), dev([t[1] for t in tiles]), dev(starts),
                         dev([p for p, _ in lens]), tabled, nq, nkv, d, scale, window, options=opts)
        close(out[many], want[many], "bfloat16", "prefill")
        if d in (64, 128) and P % 64 == 0:
            # the tcgen05 kernel: tiles of 128 rows, K and V by TMA
            out = torch.zeros_like(qd)
            assert ops.attn_prefill_tc_takes(qd, kvd, d, window)
            ops.attn_prefill_tc(qd, out, kvd, dev([t[0] for t in tiles]), dev([t[1] for t in tiles]), dev(starts),
                                dev([p for p, _ in lens]), tabled, nq, nkv, d, scale, window, options=opts)
            ops.check_tc_status(DEV)
            close(out[many], want[many], "bfloat16", "prefill on tcgen05")
    if single:
        longest = max(pos[r] for r in single) + 1
        for tma, cluster, reach in ((True, True, longest), (True, False, longest), (False, True, longest),
                                    (True, True, 64 * 40), (False, True, 64 * 40)):
            out = torch.zeros_like(qd)
            ops.DECODE_TMA, ops.DECODE_CLUSTER = tma, cluster
            try:
                ops.attn_decode(qd, out, kvd, dev(single), len(single), posd, segd, tabled, nq, nkv, d, scale, window,
                                reach, Workspace(DEV), options=opts)
            finally:
                ops.DECODE_TMA = ops.DECODE_CLUSTER = True
            close(out[single], want[single], "bfloat16", f"decode tma={tma} cluster={cluster} reach={reach}")
        ops.check_tc_status(DEV)


# ------------------------------------------------------------------- mechanisms, each alone
ALONE = {
    "attention": mz.one_layer(mz.attention(4, 2, 12, 10, 7, 6, scaling=mz.yarn(4.0, 16))),
    "attention_one_head_all_dimensions_turn_no_scaling": mz.one_layer(mz.attention(1, 1, 40, 7, 300, 40, base=77.0), streams=1),
    "attention_nothing_turns_chunk_of_one": mz.one_layer(mz.attention(2, 2, 6, 33, 1, 0), streams=2),
    "attention_value_heads_wider_than_key_heads": mz.one_layer(mz.attention(6, 3, 8, 20, 9, 4, scaling=mz.yarn(32.0, 4, 2.0, 0.5))),
    "attention_2": mz.one_layer(mz.attention_2(4, 2, 12, 10, 5, 12, 3, softcap=4.0, scaling=mz.llama3(3.0, 16))),
    "attention_2_no_convolution_no_cap": mz.one_layer(mz.attention_2(3, 1, 20, 20, 11, 8, 0), streams=4),
    "attention_2_window_of_one_long_convolution": mz.one_layer(mz.attention_2(2, 2, 10, 4, 1, 10, 6, softcap=1.0), streams=2),
    "attention_2_window_longer_than_the_sequence": mz.one_layer(mz.attention_2(5, 1, 6, 14, 400, 2, 2, softcap=100.0, scaling=mz.llama3(2.0, 8, 0.5, 3.0)), streams=1),
    "attention_2_one_tap_equal_bounds_of_the_scaling": mz.one_layer(mz.attention_2(2, 1, 12, 12, 6, 8, 1, scaling=mz.llama3(4.0, 16, 2.0, 2.0)), streams=2),
    "attention_2_nine_taps": mz.one_layer(mz.attention_2(1, 1, 16, 16, 7, 16, 9), streams=2),
    "dense_feed_forward": mz.one_layer(mz.attention(1, 1, 4, 4, 3, 2, mlp=mz.dense(40))),
    "plain_residual_no_second_table": mz.one_layer(mz.attention_2(2, 1, 8, 8, 4, 4, 2, mlp=mz.dense(24)), streams=None, bigram=None),
    "second_table_of_many_buckets": mz.one_layer(mz.attention(2, 1, 8, 8, 6, 4), bigram=(4099, 65537, 257), scale=0.3),
    "eight_streams": mz.one_layer(mz.attention(1, 1, 8, 8, 5, 8, mlp=mz.dense(24)), streams=8),
}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("what", list(ALONE))
def test_one_mechanism_alone(tmp_path, what, dtype):
    config = ALONE[what]
    state = mz.random_state(config, 31)
    folder = mz.write(str(tmp_path / "m"), config, state)
    reqs = {"a": mz.tokens(1, 41, 90), "b": mz.tokens(2, 3, 90), "c": mz.tokens(3, 1, 90)}
    want = {rid: plain.forward(config, state, toks) for rid, toks in reqs.items()}
    for cut in ("whole", "portions", "decode_tail"):
        run_and_compare(folder, config, state, reqs, CUTS[cut](reqs), dtype, 8, f"{what}, {cut}", want=want)


# --------------------------------------------------------------- whole models, every cut
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", list(mz.MZ))
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(models, which, dtype, cut):
    """Exactly as many pages as the schedule's peak needs and (mixed) four slots for five requests:
    pages and state slots are used again; free pages hold NaN."""
    reqs = requests_of(which)
    state = mz.random_state(mz.MZ[which], mz.SEEDS[which])
    run_and_compare(models[which], mz.MZ[which], state, reqs, CUTS[cut](reqs), dtype, mz.PAGE[which], f"{which} {cut}")


@pytest.mark.parametrize("which", list(mz.MZ))
def test_float32_cuts_agree_bitwise(models, which):
    """In float32 the logits at a position depend neither on the cut nor on the batch: every
    token runs the same operations in the same order whatever else the step holds."""
    reqs = requests_of(which)
    results = {}
    for cut, fn in CUTS.items():
        schedule = fn(reqs)
        engine = mz.make_engine(models[which], "float32", mz.PAGE[which], rd.peak_tokens(schedule, mz.PAGE[which]))
        results[cut] = rd.run_engine(engine, reqs, schedule)
    for cut in ("decode_tail", "portions", "mixed"):
        for rid in reqs:
            assert torch.equal(results[cut][rid], results["whole"][rid]), (cut, rid)


def test_fast_attention_kernels_take_chunks_caps_and_sinks(models, monkeypatch):
    """Configuration B in bfloat16 (heads of 64 and 128 values): decoded tokens take the split-KV
    tensor-core kernel, prompt portions the tiled one, both with chunks, windows, caps and sinks."""
    from freetoken_b200.csrc import ops
    calls = {"prefill": 0, "decode": 0}
    real_p, real_d = ops.attn_prefill, ops.attn_decode
    monkeypatch.setattr(ops, "attn_prefill", lambda *a, **k: (calls.__setitem__("prefill", 1), real_p(*a, **k))[1])
    monkeypatch.setattr(ops, "attn_decode", lambda *a, **k: (calls.__setitem__("decode", 1), real_d(*a, **k))[1])
    reqs = requests_of("B")
    state = mz.random_state(mz.MZ["B"], mz.SEEDS["B"])
    run_and_compare(models["B"], mz.MZ["B"], state, reqs, rd.mixed(reqs), "bfloat16", 64, "B mixed, fast kernels")
    assert calls == {"prefill": 1, "decode": 1}


# ------------------------------------------- the edge of a chunk, of a window; a key far back
def only_the_target_has_a_value(config, state, target, big):
    """Rewrite the value projection of the first layer so that every token of the vocabulary has next
    to no value and ``target`` a large one: whoever sees the target, with whatever weight, has an
    output that is the target's value; whoever does not has next to none.  The model has no hashed
    table, so a layer's input depends on the token alone, and the vocabulary is smaller than the
    width, so a matrix with the wanted product for every token exists.  The convolution of the values
    becomes the identity, or the target's value would reach its neighbours' rows."""
    eps = config["norm"]["eps"]
    x = state["embed"] * config["embedding"]["scale"] * state["l0.hc1.in"].sum()        # all streams equal at the start
    h = plain.layer_norm(x, state["l0.norm1"], state["l0.norm1.b"], eps)
    v = h @ state["l0.mix.v"].T
    y = 0.05 * v
    y[target] = big * v[target] / v[target].norm() * v.shape[1] ** 0.5
    state["l0.mix.v"] = torch.linalg.lstsq(h, y).solution.T.contiguous().to(torch.bfloat16).double()
    if "l0.mix.v.conv" in state:
        taps = torch.zeros_like(state["l0.mix.v.conv"])
        taps[:, -1] = 1.0
        state["l0.mix.v.conv"] = taps


def edge_layer(kind, dim, vdim, size):
    if kind == "attention":
        return mz.attention(4, 2, dim, vdim, size, dim // 2, scaling=mz.yarn(4.0, 32), mlp=mz.dense(64))
    return mz.attention_2(4, 2, dim, vdim, size, dim, 3, softcap=10.0, scaling=mz.llama3(4.0, 32), mlp=mz.dense(64))


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind,dim,page,size", [("attention", 16, 8, 24), ("attention", 64, 64, 70), ("attention", 128, 64, 64),
                                                ("attention_2", 16, 8, 24), ("attention_2", 64, 64, 129), ("attention_2", 128, 64, 64)])
def test_an_edge_decides(tmp_path, kind, dim, page, size, dtype):
    """The asking position sees its target ``size - 1`` positions back (a window) or at the first
    position of its own chunk, and must not see it one position further back; asked from inside a
    prompt portion and by a decoded token; chunks and windows shorter than, equal to and longer than a
    page; pages behind them are given back while the requests run (heads of 16 values: the generic
    kernel, of 64 and 128 the tensor-core kernels in bfloat16)."""
    config = mz.one_layer(edge_layer(kind, dim, dim if dim > 16 else 12, size), vocab=40, width=48, streams=2, bigram=None)
    state = mz.random_state(config, 41)
    target, stand_in = 7, 13
    only_the_target_has_a_value(config, state, target, big=40.0)
    n = 330
    reqs = {}
    for name, back in (("inside", size - 1), ("outside", size), ("next_to", 1), ("far_outside", 2 * size + 3)):
        toks = [t if t != target else stand_in for t in mz.tokens(60 + back, n, 40)]
        for at in (n - 40, n - 1):            # asked from a prompt portion and by the last decoded token
            if kind == "attention":
                at = at // size * size + size - 1 if at // size * size + size - 1 < n else at // size * size - 1
            toks[at - back] = target
        reqs[name] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    blind = [t if t != target else stand_in for t in reqs["inside"]]
    diff = mz.position_errors(plain.forward(config, state, blind), want["inside"])
    assert float(diff.max()) > 0.2
    folder = mz.write(str(tmp_path / "m"), config, state)
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = mz.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        mz.compare(rd.run_engine(engine, reqs, schedule), want, mz.TOL[dtype], f"{kind} {size}, {cut} [{dtype}]")
        assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_a_far_key_decides(tmp_path, kind, dtype):
    """One key among hundreds, 300 to 450 positions back inside a chunk of 512 (a window of 500),
    right before, on and right after a page border and first of all: it alone has a value, and the
    output projection is made twelve times as large, so that a weight of 1/450 on that value moves
    the logits.  In bfloat16 the other tokens' small values are differences of products of the
    rounded input and come out up to 0.08 off whatever computes them (which is also why the
    vocabulary is a quarter of the width here, and why the value is not simply made larger); with
    the softmax whose sink is only 1, where a token's own value keeps much of the weight, that shows
    as an error of up to 0.18 at some tokens, so the bound there is 0.2 - less than a third of what
    losing the far key costs."""
    size = 512 if kind == "attention" else 500
    config = mz.one_layer(edge_layer(kind, 16, 12, size), vocab=12, width=48, streams=2, bigram=None)
    state = mz.random_state(config, 43)
    target, stand_in = 5, 6
    only_the_target_has_a_value(config, state, target, big=40.0)
    state["l0.mix.o"] = (state["l0.mix.o"] * 12.0).to(torch.bfloat16).double()
    page, n = 16, 470
    reqs = {}
    for place in (15, 16, 17, 0, 145):
        toks = [t if t != target else stand_in for t in mz.tokens(70 + place, n, 12)]
        toks[place] = target
        reqs[f"t{place}"] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    other = list(reqs["t16"])
    other[16] = stand_in
    tol = 0.2 if (kind, dtype) == ("attention", "bfloat16") else mz.TOL[dtype]
    assert float(mz.position_errors(plain.forward(config, state, other)[-1:], want["t16"][-1:])) > max(0.2, 3 * tol)
    folder = mz.write(str(tmp_path / "m"), config, state)
    for cut in ("decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = mz.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        mz.compare(rd.run_engine(engine, reqs, schedule), want, tol, f"far key, {kind}, {cut} [{dtype}]")


# ------------------------------------------------- long prompts at sizes between tiny and real
LONG = mz.model(640, 256, 2, 1e-5, [
    mz.attention(4, 2, 64, 64, 200, 32, base=40000.0, scaling=mz.yarn(6.0, 256), mlp=mz.dense(512)),
    mz.attention_2(4, 2, 64, 32, 64, 64, 4, softcap=15.0, base=2e6, scaling=mz.llama3(5.0, 512), mlp=mz.dense(384)),
    mz.attention(8, 1, 32, 64, 1024, 16, base=500.0, mlp=mz.dense(256)),
    mz.attention_2(2, 2, 128, 128, 700, 64, 3, softcap=45.0, base=1e5, scaling=mz.llama3(4.0, 128, 1.0, 8.0)),
], scale=16.0, bigram=(8191, 131, 17), loop=(1, 3, 2))


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_prompts(tmp_path, dtype):
    """Prompts of up to 1,500 tokens (two dozen pages of 64, chunks and windows that pass many of them,
    positions beyond the length the frequency scaling starts from, heads of 64 and 128 values on the
    tensor-core kernels in bfloat16), whole and in a mixed batch whose decoded tokens read hundreds of keys."""
    state = mz.random_state(LONG, 7)
    folder = mz.write(str(tmp_path / "m"), LONG, state)
    reqs = {f"r{i}": mz.tokens(11 * i + 3, n, LONG["vocab"]) for i, n in enumerate([1500, 700, 64, 65, 129])}
    want = {rid: plain.forward(LONG, state, toks) for rid, toks in reqs.items()}
    for cut in ("whole", "mixed"):
        run_and_compare(folder, LONG, state, reqs, CUTS[cut](reqs), dtype, 64, f"long {cut}", want=want)


# --------------------------------------------------------- first tokens, long decoding
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", ["A", "B"])
def test_first_tokens_and_long_decoding(models, which, dtype):
    """A request that starts with a single token and is decoded one token at a time for 200 steps (chunks
    end, windows pass, pages go back, decode steps are replayed from a graph in bfloat16), beside a second
    request that joins later two tokens a step; against the whole sequences."""
    from freetoken_b200.engine import StepEntry
    config = mz.MZ[which]
    state = mz.random_state(config, mz.SEEDS[which])
    a, b = mz.tokens(5, 201, config["vocab"]), mz.tokens(6, 120, config["vocab"])
    page = mz.PAGE[which]
    engine = mz.make_engine(models[which], dtype, page, 2 * page + 204 + 120)
    got_a, got_b = [], []
    for i in range(len(a)):
        entries = [StepEntry("a", [a[i]], [0])]
        j = i - 60
        if 0 <= j < len(b) // 2:
            entries.append(StepEntry("b", b[2 * j:2 * j + 2], [0, 1]))
        logits = engine.step(entries).float().cpu()
        got_a.append(logits[0])
        got_b.extend(logits[1:])
    want = {"a": plain.forward(config, state, a), "b": plain.forward(config, state, b)}
    mz.compare({"a": torch.stack(got_a), "b": torch.stack(got_b)}, want, mz.TOL[dtype], f"long decoding [{dtype}]")
    if dtype == "bfloat16":
        assert engine.graph_replays > 0


# ------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", ["A", "B", "D"])
def test_greedy_generation_through_the_scheduler(models, which, dtype):
    """``LLM.generate`` (scheduler, overlapped steps - a decoded token's predecessor is still on the device
    when the next step is planned -, graph replay of decode steps in bfloat16): every generated token is the
    plain model's own greedy choice for the sequence so far, unless its two best logits lie within rounding
    of each other."""
    from freetoken_b200 import LLM, SamplingParams
    config = mz.MZ[which]
    state = mz.random_state(config, mz.SEEDS[which])
    llm = LLM(models[which], dtype, page_size=mz.PAGE[which], num_token_override=1024, max_running_req=3,
              max_extend_tokens=24)
    prompts = [mz.tokens(70 + i, n, config["vocab"]) for i, n in enumerate((3, 30, 11, 1, 47))]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    tie = 1e-4 if dtype == "float32" else 8e-2
    ties = 0
    for prompt, result in zip(prompts, out):
        seq = list(prompt)
        assert len(result["token_ids"]) == 12
        for token in result["token_ids"]:
            logits = plain.forward(config, state, seq)[-1]
            if token != int(logits.argmax()):
                assert float(logits.max() - logits[token]) < tie, (dtype, len(seq), token, int(logits.argmax()))
                ties += 1
            seq.append(int(token))
    assert ties == 0 if dtype == "float32" else ties <= 4
    if dtype == "bfloat16":
        assert llm.engine.graph_replays > 0


# -------------------------------------------------------------------- the replay tool
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_trace_replay_tool(models, tmp_path, dtype):
    """``bin/trace_run`` on a Mezapel folder: a mixed schedule with exactly the pages its peak needs."""
    which = "A"
    reqs = requests_of(which)
    state = mz.random_state(mz.MZ[which], mz.SEEDS[which])
    schedule = rd.mixed(reqs)
    page = mz.PAGE[which]
    got = rd.run_trace_tool(models[which], dtype, reqs, schedule, str(tmp_path / "out"),
                            rd.peak_tokens(schedule, page), page, mz.MZ[which]["vocab"])
    want = {rid: plain.forward(mz.MZ[which], state, toks) for rid, toks in reqs.items()}
    mz.compare(got, want, mz.TOL[dtype], f"trace_run, mixed [{dtype}]")


# ------------------------------------------- heads of sizes the tensor-core kernels do not take
FILLED = mz.model(200, 160, 2, 1e-5, [
    mz.attention(4, 2, 80, 48, 300, 40, base=20000.0, scaling=mz.yarn(4.0, 128), mlp=mz.dense(256)),
    mz.attention_2(4, 1, 40, 72, 90, 40, 3, softcap=25.0, scaling=mz.llama3(4.0, 256), mlp=mz.dense(192)),
], scale=12.0, bigram=(251, 13, 29))


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_heads_of_other_sizes_are_filled_up_for_the_tensor_core_kernels(tmp_path, monkeypatch, dtype):
    """Heads of 80 (keys) and 48 (values), of 40 and 72: in bfloat16 the mixer fills them up to 128 and
    runs prompts on the tcgen05 and mma.sync kernels and decoded tokens on the split-KV kernel; the norm
    over q and k still counts the real values only.  float32 keeps heads of 80 and 72 on the generic kernel."""
    from freetoken_b200.csrc import ops
    calls = {"prefill": 0, "prefill_tc": 0, "decode": 0, "generic": 0}
    for name, fn in (("prefill", "attn_prefill"), ("prefill_tc", "attn_prefill_tc"), ("decode", "attn_decode"),
                     ("generic", "attn_paged_simt")):
        real = getattr(ops, fn)
        monkeypatch.setattr(ops, fn, lambda *a, _n=name, _r=real, **k: (calls.__setitem__(_n, calls[_n] + 1), _r(*a, **k))[1])
    state = mz.random_state(FILLED, 9)
    folder = mz.write(str(tmp_path / "m"), FILLED, state)
    reqs = {f"r{i}": mz.tokens(17 * i + 1, n, FILLED["vocab"]) for i, n in enumerate([700, 130, 64, 3])}
    want = {rid: plain.forward(FILLED, state, toks) for rid, toks in reqs.items()}
    for cut in ("whole", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = mz.make_engine(folder, dtype, 64, rd.peak_tokens(schedule, 64), poison=True)
        sizes = [b.mixer.d for b in engine.model.blocks]
        assert sizes == ([128, 128] if dtype == "bfloat16" else [80, 72])
        mz.compare(rd.run_engine(engine, reqs, schedule), want, mz.TOL[dtype], f"filled heads, {cut} [{dtype}]")
    if dtype == "bfloat16":
        assert calls["generic"] == 0 and min(calls["prefill"], calls["prefill_tc"], calls["decode"]) > 0, calls
    else:
        assert calls["generic"] > 0 and calls["prefill"] + calls["prefill_tc"] + calls["decode"] == 0, calls
