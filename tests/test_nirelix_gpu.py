"""Nirelix in the engine against the plain implementation: every new kernel alone, every mechanism
alone in a one-layer model, whole prompts against decoding, portions down to two tokens, mixed
batches with pages and state slots used again, a window's edge and a token far back made decisive
on purpose, the first tokens, long decoding, three configurations that differ in every size,
greedy generation through the scheduler, the trace replay tool."""

import pytest
import torch

import nirelix_tiny as nx
import plain_nirelix as plain
import replay_driver as rd

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 2, 9, 37, 70], "B": [3, 150, 66, 260, 21], "C": [2, 35, 77, 5]}
CUTS = {"whole": rd.whole, "decode_tail": rd.decode_tail, "portions": rd.portions, "mixed": rd.mixed}
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def requests_of(which):
    vocab = nx.NX[which]["vocab"]
    return {f"r{i}": nx.tokens(30 * i + ord(which), n, vocab) for i, n in enumerate(LENGTHS[which])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {which: nx.write_tiny(str(tmp_path_factory.mktemp(f"nx{which}")), which) for which in nx.NX}


def expected_for(config, state, reqs, dtype, routing=None):
    """The plain model's logits; in bfloat16 with the experts the engine chose (two correct
    implementations may choose differently where two router scores lie within rounding)."""
    out = {}
    routed = nx.routed_layers(config)
    for rid, toks in reqs.items():
        ids = dict(zip(routed, routing[rid])) if dtype == "bfloat16" and routing else None
        out[rid] = plain.forward(config, state, toks, expert_ids=ids)
    return out


def run_engine(engine, reqs, schedule, routing=None):
    """Drive ``engine.step`` through a schedule; logits of every position of every request.  With
    ``routing`` (a dict) the experts the engine chose are left there: ``routing[request][j]`` is
    ``[positions, top]`` of the j-th routed layer."""
    from freetoken_b200.engine import StepEntry
    out = {rid: torch.full((len(t), engine.vocab_size), float("nan")) for rid, t in reqs.items()}
    for entries, ended in schedule:
        batch = [StepEntry(rid, reqs[rid][first:first + n], list(range(n))) for rid, first, n in entries]
        probe = {"router_ids": []} if routing is not None else None
        logits = engine.step(batch, probe=probe).float().cpu()
        row = 0
        for rid, first, n in entries:
            out[rid][first:first + n] = logits[row:row + n]
            if routing is not None:
                if rid not in routing:
                    routing[rid] = [torch.full((len(reqs[rid]), x.shape[1]), -1, dtype=torch.long)
                                    for x in probe["router_ids"]]
                for j, x in enumerate(probe["router_ids"]):
                    routing[rid][j][first:first + n] = x[row:row + n].cpu().long()
            row += n
        for rid in ended:
            engine.end_request(rid)
    engine.cache.check_integrity()
    return out


def run_and_compare(folder, config, state, reqs, schedule, dtype, page, what, tol=None, poison=True):
    engine = nx.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=poison)
    routing = {} if nx.routed_layers(config) else None
    got = run_engine(engine, reqs, schedule, routing)
    want = expected_for(config, state, reqs, dtype, routing)
    nx.compare(got, want, tol or nx.TOL[dtype], f"{what} [{dtype}]")
    assert engine.cache.free_pages() == engine.cache.total_pages()
    return got


def close(got, want, dtype, what=""):
    tol = 2e-5 if dtype == "float32" else 2e-2
    g, w = got.double().cpu(), want.double()
    assert torch.allclose(g, w, atol=tol * max(1.0, float(w.abs().max())), rtol=tol), (what, float((g - w).abs().max()))


# ------------------------------------------------------------------ kernels, each alone
def segments(lens, slots, pos0=None):
    q = [0]
    for n in lens:
        q.append(q[-1] + n)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int().cuda()
    out = [seg, torch.tensor(slots, dtype=torch.int32).cuda(), torch.tensor(q, dtype=torch.int32).cuda()]
    if pos0 is not None:
        out.append(torch.tensor(pos0, dtype=torch.int32).cuda())
    return out


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("S,H,k", [(1, 40, 1), (2, 70, 3), (3, 200, 1), (4, 1030, 2), (8, 64, 1), (4, 2048, 2), (2, 4104, 1), (1, 520, 3)])
def test_hyper_norm(dtype, S, H, k):
    """A pending branch of k partial rows joins S streams, the next input is formed and layer-normed;
    without a branch nothing is written; without read weights the plain sum is normed."""
    from freetoken_b200.csrc import ops
    torch.manual_seed(S * 100 + k)
    T = 5
    x = torch.randn(T, S, H)
    y = torch.randn(T, k, H).to(DTYPES[dtype])
    mix, out_w, read = torch.randn(S, S), torch.randn(S), torch.randn(S)
    weight, bias = torch.randn(H), torch.randn(H)
    streams = x.cuda().clone()
    normed = torch.empty(T, H, dtype=DTYPES[dtype], device="cuda")
    ops.hyper_norm(streams, y.cuda() if k > 1 else y[:, 0].contiguous().cuda(), mix.cuda(), out_w.cuda(), read.cuda(),
                   weight.cuda(), bias.cuda(), 1e-5, True, normed)
    xs = x.double().permute(1, 0, 2)                                       # [S, T, H]
    new = torch.einsum("sr,sth->rth", mix.double(), xs) + out_w.double()[:, None, None] * y.double().sum(1)[None]
    close(streams.permute(1, 0, 2), new, "float32", "streams")
    u = torch.einsum("s,sth->th", read.double(), new)
    close(normed, plain.layer_norm(u, weight.double(), bias.double(), 1e-5), dtype, "normed")
    # no branch: the streams stay, the plain sum is RMS-normed without a bias
    before = streams.clone()
    ops.hyper_norm(streams, None, None, None, None, weight.cuda(), None, 1e-5, False, normed)
    assert torch.equal(streams, before)
    close(normed, plain.rms(before.double().cpu().sum(1), 1e-5) * weight.double(), dtype, "sum, rms")


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_rows_embedding_copies_rms_rows_clamped_pair_sigmoid_gate(dtype):
    from freetoken_b200.csrc import ops
    torch.manual_seed(3)
    dt = DTYPES[dtype]
    table = torch.randn(20, 36).to(torch.bfloat16).cuda()
    ids = torch.tensor([3, 19, 0], dtype=torch.int32).cuda()
    res = torch.empty(3, 4, 36, device="cuda")
    ops.embed_gather(ids, table, res)
    assert torch.equal(res, table.float()[ids.long()][:, None, :].expand(3, 4, 36))
    wide = torch.randn(7, 50).to(dt).cuda()
    w = torch.randn(22).cuda()
    out = torch.zeros(7, 30, dtype=dt, device="cuda")
    ops.rms_rows(wide[:, 9:31], w, out[:, 4:26], 1e-4)
    close(out[:, 4:26], plain.rms(wide[:, 9:31].double().cpu(), 1e-4) * w.double().cpu(), dtype, "rms_rows")
    assert float(out[:, :4].abs().max()) == 0 and float(out[:, 26:].abs().max()) == 0
    gu = (3 * torch.randn(6, 2 * 22)).to(dt).cuda()
    mid = torch.empty(6, 22, dtype=dt, device="cuda")
    ops.glu_rows(gu, mid, "swigluoai", 1.702, 1.5)
    g = gu[:, :22].double().cpu().clamp(max=1.5)
    u = gu[:, 22:].double().cpu().clamp(-1.5, 1.5)
    close(mid, g * torch.sigmoid(1.702 * g) * (u + 1), dtype, "clamped pair")
    y = torch.randn(6, 48).cuda()
    gate = torch.randn(6, 48).to(dt).cuda()
    nw = torch.randn(12).cuda()
    out = torch.empty(6, 48, dtype=dt, device="cuda")
    ops.gated_norm(y, gate, nw, out, 4, 1e-5, gate_first=False, gate_kind="sigmoid")
    want = plain.rms(y.double().cpu().view(6, 4, 12), 1e-5) * nw.double().cpu() * torch.sigmoid(gate.double().cpu()).view(6, 4, 12)
    close(out, want.reshape(6, 48), dtype, "sigmoid gate")


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("heads,dq,rank,rot,page", [(3, 5, 18, 4, 4), (2, 16, 32, 32, 8), (1, 7, 6, 2, 3)])
def test_latent_store(dtype, heads, dq, rank, rot, page):
    """The normed latent and the rotated key part land in the token's place of its page, the rotated tail
    of every head's query behind the first rank values of its absorbed row; two requests whose pages
    interleave, positions across page borders."""
    from freetoken_b200.csrc import ops
    from freetoken_b200.parts.position import rotary_table
    torch.manual_seed(rank)
    dt = DTYPES[dtype]
    lens, pos0 = [5, 3], [page - 2, 2 * page - 1]
    T = sum(lens)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int()
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(pos0, lens)]).int()
    table = torch.tensor([[1, 4, 2, 7], [6, 3, 5, 8]], dtype=torch.int32)
    down = torch.randn(T, rank + rot + 3).to(dt)
    q = torch.randn(T, heads * (dq + rot)).to(dt)
    w = torch.randn(rank)
    pages = torch.zeros(9, 1, page, rank + rot, dtype=dt, device="cuda")
    q_abs = torch.zeros(T, heads, rank + rot, dtype=dt, device="cuda")
    cs = rotary_table(rot, 77.0, "cuda", 64, exact_angles=True)
    ops.latent_store(down.cuda()[:, 2:2 + rank + rot], q.cuda(), q_abs, pages, w.cuda(), cs, pos.cuda(), seg.cuda(),
                     table.cuda(), heads=heads, q_dim=dq, rank=rank, rot=rot, interleaved=True, eps=1e-5)
    d = down[:, 2:2 + rank + rot].double()
    for t in range(T):
        p = int(pos[t])
        row = pages[int(table[int(seg[t]), p // page]), 0, p % page].cpu()
        close(row[:rank], plain.rms(d[t, :rank], 1e-5) * w.double(), dtype, "latent")
        close(row[rank:], plain.rotate_pairs(d[t, rank:].view(1, 1, rot), 77.0, rot, first=p)[0, 0], dtype, "key part")
        qt = plain.rotate_pairs(q[t].double().view(1, heads, dq + rot)[..., dq:], 77.0, rot, first=p)[0]
        close(q_abs[t, :, rank:], qt, dtype, "query tails")
    assert float(q_abs[:, :, :rank].abs().max()) == 0
    assert int((pages.abs().sum(-1) > 0).sum()) == T


def plain_retention_rows(q, k, v, decay, rot, base, D):
    T, H = q.shape[0], len(decay)
    qr = plain.rotate_halves(q, base, rot) if rot else q
    kr = (plain.rotate_halves(k, base, rot) if rot else k) * D ** -0.5
    out = torch.zeros(T, H, v.shape[-1], dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(D, v.shape[-1], dtype=torch.float64)
        for t in range(T):
            S = decay[h] * S + torch.outer(kr[t, h], v[t, h])
            out[t, h] = S.T @ qr[t, h]
    return out


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,D,P,rot", [(2, 12, 5, 6), (3, 40, 70, 40), (1, 64, 32, 0), (2, 200, 9, 64)])
def test_retention_scan_in_segments(dtype, H, D, P, rot):
    """Two requests fed in segments of 1 to 19 tokens that interleave, in slots 2 and 0: every read-out
    equals the recurrence over the whole sequence (positions continue across segments)."""
    from freetoken_b200.csrc import ops
    from freetoken_b200.parts.position import rotary_table
    torch.manual_seed(D)
    dt = DTYPES[dtype]
    n = 45
    decay = [0.9, 0.999, 0.5][:H]
    rows = {r: torch.randn(n, 2 * H * D + H * P).to(dt) for r in ("a", "b")}
    want = {}
    for r, x in rows.items():
        xd = x.double()
        want[r] = plain_retention_rows(xd[:, :H * D].view(n, H, D), xd[:, H * D:2 * H * D].view(n, H, D),
                                       xd[:, 2 * H * D:].view(n, H, P), decay, rot, 1000.0, D).reshape(n, H * P)
    state = torch.zeros(4, H * D * P + 3, device="cuda")
    state[:, H * D * P:] = 7.0
    cs = rotary_table(rot, 1000.0, "cuda", 64, exact_angles=True) if rot else None
    at = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    for step, cut in enumerate([(1, 3), (2, 1), (9, 2), (1, 1), (13, 19), (19, 19)]):
        order = ("a", "b") if step % 2 == 0 else ("b", "a")
        lens = [cut[0] if r == "a" else cut[1] for r in order]
        x = torch.cat([rows[r][at[r]:at[r] + m] for r, m in zip(order, lens)]).cuda()
        seg, slot, qs, p0 = segments(lens, [2 if r == "a" else 0 for r in order], [at[r] for r in order])
        o = torch.empty(x.shape[0], H * P, device="cuda")
        ops.retention_scan(x, torch.tensor(decay).cuda(), cs, p0, state[:, :H * D * P], o, slot, qs, H, D, P, D ** -0.5)
        o = o.cpu()
        for r, m in zip(order, lens):
            got[r].append(o[:m])
            o = o[m:]
            at[r] += m
    for r in rows:
        g = torch.cat(got[r]).double()
        scale = float(want[r].abs().max())
        assert float((g - want[r]).abs().max()) < (3e-5 if dtype == "float32" else 2e-2) * scale, r
    assert float(state[1, :H * D * P].abs().max()) == 0 and bool((state[:, H * D * P:] == 7.0).all())


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,G,D,P", [(4, 2, 12, 10), (2, 2, 40, 70), (3, 1, 64, 8), (1, 1, 200, 12)])
def test_channel_delta_scan_in_segments(dtype, H, G, D, P):
    """The delta rule with a decay per key channel, cut into segments below, at and above a chunk."""
    from freetoken_b200.csrc import ops
    torch.manual_seed(D + P)
    dt = DTYPES[dtype]
    n = 45
    qkv = torch.randn(n, 2 * G * D + H * P).to(dt)
    beta = torch.randn(n, H).to(dt)
    a = torch.randn(n, H * D)
    a_log, dt_bias = torch.randn(H) - 1.0, torch.randn(H * D) - 0.5
    x = qkv.double()
    q, k, v = x[:, :G * D].view(n, G, D), x[:, G * D:2 * G * D].view(n, G, D), x[:, 2 * G * D:].view(n, H, P)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    g = torch.exp(-torch.exp(a_log.double())[None, :, None] * plain.softplus(a.double() + dt_bias.double()).view(n, H, D))
    b = torch.sigmoid(beta.double())
    want = torch.zeros(n, H, P, dtype=torch.float64)
    for h in range(H):
        S = torch.zeros(D, P, dtype=torch.float64)
        for t in range(n):
            S = g[t, h][:, None] * S
            u = b[t, h] * (v[t, h] - S.T @ k[t, h // (H // G)])
            S = S + torch.outer(k[t, h // (H // G)], u)
            want[t, h] = S.T @ q[t, h // (H // G)]
    state = torch.zeros(3, H * D * P, device="cuda")
    got, at = [], 0
    for m in (1, 7, 8, 9, 2, 18):
        seg, slot, qs = segments([m], [1])
        o = torch.empty(m, H * P, device="cuda")
        ops.channel_delta_scan(qkv[at:at + m].cuda(), beta[at:at + m].cuda(), a[at:at + m].cuda(), dt_bias.cuda(),
                               a_log.cuda(), state, o, slot, qs, H, G, D, P, 1e-6, D ** -0.5)
        got.append(o.cpu())
        at += m
    g_ = torch.cat(got).double()
    scale = float(want.abs().max())
    assert float((g_ - want.view(n, H * P)).abs().max()) < (3e-5 if dtype == "float32" else 2e-2) * scale
    assert float(state[0].abs().max()) == 0 and float(state[2].abs().max()) == 0


@pytest.mark.parametrize("E,top,count,keep", [(8, 3, 4, 3), (6, 2, 3, 1), (12, 4, 1, 1), (9, 2, 9, 4), (64, 6, 8, 2), (5, 5, 5, 5)])
def test_router_chooses_inside_the_best_groups(E, top, count, keep):
    """Both selection kernels against the plain choice: groups of one, two and more experts, one, some
    and all groups kept, negative choice scores (a dropped group counts as minus infinity, not 0)."""
    from freetoken_b200.csrc import ops
    torch.manual_seed(E)
    for T in (5, 70):
        logits = torch.randn(T, E) * 2
        bias = torch.randn(E) - 1.5                       # most choice scores negative
        w = {"r.router": torch.eye(E, dtype=torch.float64), "r.correction": bias.double()}
        router = {"experts": E, "top": top, "scale": 2.5, "groups": {"count": count, "keep": keep}}
        want_ids, want_w = plain.choose_experts(logits.double(), w, "r.", router)
        ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
        weights = torch.empty(T, top, device="cuda")
        ops.router_select(logits.cuda(), bias.cuda(), ids, weights, top, False, True, 2.5, 1, count, keep)
        assert torch.equal(ids.cpu().long().sort(1).values, want_ids.sort(1).values)
        order = ids.cpu().long().argsort(1), want_ids.argsort(1)
        assert torch.allclose(weights.cpu().double().gather(1, order[0]), want_w.gather(1, order[1]), atol=1e-5)
        if ops.route_small_takes(T, E, top):
            R = T * top
            bufs = [torch.empty(n, dtype=torch.int32, device="cuda") for n in (E, E + 1, R, R, E + 1)]
            ids2 = torch.empty(T, top, dtype=torch.int32, device="cuda")
            w2 = torch.empty(T, top, device="cuda")
            ops.route_small(logits.cuda(), bias.cuda(), ids2, w2, *bufs, top, False, True, 2.5, 1, count, keep)
            assert torch.equal(ids2, ids) and torch.equal(w2, weights)


# ------------------------------------------------------------------- mechanisms, each alone
ALONE = {
    "retention": nx.one_layer(nx.retention(3, 12, 10, (0.9, 0.99, 0.7), 8)),
    "retention_all_dimensions_turn_one_head": nx.one_layer(nx.retention(1, 40, 7, (0.995,), 40, base=77.0), streams=1),
    "retention_nothing_turns": nx.one_layer(nx.retention(2, 6, 33, (1.0, 0.25), 0), streams=2),
    "channel_delta": nx.one_layer(nx.channel_delta(4, 2, 12, 10, 3, 6)),
    "channel_delta_one_key_head_no_memory_of_inputs": nx.one_layer(nx.channel_delta(3, 1, 40, 7, 1, 2), streams=4),
    "latent_attention": nx.one_layer(nx.latent(3, 8, 6, 10, 20, 14, 5)),
    "latent_attention_one_head_long_window": nx.one_layer(nx.latent(1, 4, 12, 20, 7, 30, 300, base=50.0), streams=1),
    "latent_attention_window_of_one": nx.one_layer(nx.latent(4, 10, 2, 3, 9, 5, 1, scale=0.7), streams=2),
    "latent_attention_rows_wider_than_512": nx.one_layer(nx.latent(2, 8, 8, 6, 10, 520, 9), streams=2),
    "dense_feed_forward": nx.one_layer(nx.retention(1, 4, 4, (0.9,), 2, mlp=nx.dense(40, 0.7))),
    "routed_feed_forward": nx.one_layer(nx.retention(1, 4, 4, (0.9,), 2, mlp=nx.moe(8, 3, 16, 4, 2, scale=2.5))),
    "routed_feed_forward_top_one_no_groups": nx.one_layer(nx.retention(1, 4, 4, (0.9,), 2, mlp=nx.moe(4, 1, 16, 1, 1)), streams=1),
    "eight_streams": nx.one_layer(nx.channel_delta(1, 1, 8, 8, 2, 4, nx.dense(24, 2.0)), streams=8),
}


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("what", list(ALONE))
def test_one_mechanism_alone(tmp_path, what, dtype):
    config = ALONE[what]
    state = nx.random_state(config, 31)
    folder = nx.write(str(tmp_path / "m"), config, state)
    reqs = {"a": nx.tokens(1, 41, 90), "b": nx.tokens(2, 3, 90), "c": nx.tokens(3, 1, 90)}
    for cut in ("whole", "portions", "decode_tail"):
        run_and_compare(folder, config, state, reqs, CUTS[cut](reqs), dtype, 8, f"{what}, {cut}")


# --------------------------------------------------------------- whole models, every cut
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", list(nx.NX))
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(models, which, dtype, cut):
    """Exactly as many pages as the schedule's peak needs and (mixed) four slots for five requests:
    pages and state slots are used again; free pages hold NaN."""
    reqs = requests_of(which)
    state = nx.random_state(nx.NX[which], nx.SEEDS[which])
    run_and_compare(models[which], nx.NX[which], state, reqs, CUTS[cut](reqs), dtype, nx.PAGE[which], f"{which} {cut}")


@pytest.mark.parametrize("which", list(nx.NX))
def test_float32_cuts_agree_bitwise(models, which):
    """In float32 the logits at a position depend neither on the cut nor on the batch: every
    token runs the same operations in the same order whatever else the step holds."""
    reqs = requests_of(which)
    results = {}
    for cut, fn in CUTS.items():
        schedule = fn(reqs)
        engine = nx.make_engine(models[which], "float32", nx.PAGE[which], rd.peak_tokens(schedule, nx.PAGE[which]))
        results[cut] = run_engine(engine, reqs, schedule)
    for cut in ("decode_tail", "portions", "mixed"):
        for rid in reqs:
            assert torch.equal(results[cut][rid], results["whole"][rid]), (cut, rid)


def test_fast_attention_kernels_take_the_latent_rows(models, monkeypatch):
    """Configuration B in bfloat16 (cached rows of 64 and 128 values): decoded tokens take the split-KV
    tensor-core kernel, prompt portions the tiled one, both with windows."""
    from freetoken_b200.csrc import ops
    calls = {"prefill": 0, "decode": 0}
    real_p, real_d = ops.attn_prefill, ops.attn_decode
    monkeypatch.setattr(ops, "attn_prefill", lambda *a, **k: (calls.__setitem__("prefill", 1), real_p(*a, **k))[1])
    monkeypatch.setattr(ops, "attn_decode", lambda *a, **k: (calls.__setitem__("decode", 1), real_d(*a, **k))[1])
    reqs = requests_of("B")
    state = nx.random_state(nx.NX["B"], nx.SEEDS["B"])
    run_and_compare(models["B"], nx.NX["B"], state, reqs, rd.mixed(reqs), "bfloat16", 64, "B mixed, fast kernels")
    assert calls == {"prefill": 1, "decode": 1}


# ------------------------------------------------------------ a window's edge, sharp on purpose
def sharpen_latent(config, state, asker, target, beta):
    """Rewrite the query up-projection of the first layer so that token ``asker``'s unrotated query is
    ``beta`` times token ``target``'s unrotated key in every head and its rotated part is zero:
    wherever ``target`` stands inside the window, ``asker`` puts nearly all its weight there, whatever
    the distance (the rotated parts, which depend on it, are silenced)."""
    m = config["layers"][0]["mixer"]
    H, D, R = m["heads"], m["dim"], m["rot_dim"]
    eps = config["norm"]["eps"]
    x = state["embed"][[asker, target]] * state["l0.hc1.in"].sum()             # all streams equal at the start
    h = plain.layer_norm(x, state["l0.norm1"], state["l0.norm1.b"], eps)
    cq = plain.rms(state["l0.mix.dq"] @ h[0], eps) * state["l0.mix.dq.norm"]
    c = plain.rms((state["l0.mix.dkv"] @ h[1])[:m["kv_rank"]], eps) * state["l0.mix.dkv.norm"]
    k = (state["l0.mix.uk"] @ c).view(H, D)
    want = torch.cat([beta * k, torch.zeros(H, R, dtype=torch.float64)], dim=1).reshape(H * (D + R))
    uq = state["l0.mix.uq"]
    uq = uq - (uq @ cq)[:, None] * cq[None, :] / cq.dot(cq) + want[:, None] * cq[None, :] / cq.dot(cq)
    state["l0.mix.uq"] = uq.to(torch.bfloat16).double()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("dim,rot,rank,page,window", [(16, 8, 20, 8, 24), (32, 16, 48, 64, 70), (16, 32, 96, 64, 64), (64, 16, 112, 64, 129)])
def test_a_window_edge_decides(tmp_path, dim, rot, rank, page, window, dtype):
    """The asking token finds its target ``window - 1`` tokens back and must not find it ``window`` back,
    inside a prompt portion and as a decoded token; windows shorter than, equal to and longer than a
    page; pages the window has passed are given back while the requests run (cached rows of 28 values:
    the generic kernel, of 64 and 128 the tensor-core kernels in bfloat16)."""
    config = nx.one_layer(nx.latent(2, dim, rot, 12, 20, rank, window, scale=0.25), vocab=120, width=48, streams=2)
    state = nx.random_state(config, 41)
    asker, target = 7, 11
    sharpen_latent(config, state, asker, target, beta=160.0 / dim)
    n = 330
    reqs = {}
    for name, back in (("inside", window - 1), ("outside", window), ("next_to", 1), ("far_outside", 2 * window + 3)):
        toks = [t if t not in (asker, target) else 13 for t in nx.tokens(60 + back, n, 120)]
        for at in (n - 40, n - 1):            # asked from a prompt portion and by the last decoded token
            toks[at] = asker
            toks[at - back] = target
        reqs[name] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    blind = [t if t != target else 13 for t in reqs["inside"]]
    assert float(nx.position_errors(plain.forward(config, state, blind)[-1:], want["inside"][-1:])) > 0.2
    folder = nx.write(str(tmp_path / "m"), config, state)
    tol = nx.TOL[dtype] * (1 if dtype == "float32" else 2)      # a sharp softmax: rounding of scores counts more
    for cut in ("whole", "decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = nx.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        nx.compare(run_engine(engine, reqs, schedule), want, tol, f"window {window}, {cut} [{dtype}]")
        assert engine.cache.free_pages() == engine.cache.total_pages()


# ------------------------------------------------------- a token far back, through the state
def only_the_target_writes(config, state, target, kind):
    """Rewrite the projection that sets how much a token writes into the state so that every token of the
    vocabulary writes next to nothing and ``target`` writes fully: the delta rule's write strength,
    or (retention, which has none) the value projection itself.  The vocabulary is smaller than the
    width, so a matrix with the wanted product for every token exists."""
    eps = config["norm"]["eps"]
    h = plain.layer_norm(state["embed"] * state["l0.hc1.in"].sum(), state["l0.norm1"], state["l0.norm1.b"], eps)
    if kind == "channel_delta":
        y = torch.full((h.shape[0],), -7.0, dtype=torch.float64)
        y[target] = 3.0
        row = torch.linalg.lstsq(h, y[:, None]).solution[:, 0]
        heads = config["layers"][0]["mixer"]["heads"]
        state["l0.mix.b"] = row.repeat(heads, 1).to(torch.bfloat16).double()
    else:
        v = state["l0.mix.v"]
        y = 0.05 * (h @ v.T)                                   # everybody's values shrink ...
        y[target] = 3.0 * (h[target] @ v.T)                    # ... but the target's grow
        state["l0.mix.v"] = torch.linalg.lstsq(h, y).solution.T.contiguous().to(torch.bfloat16).double()


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("kind", ["retention", "channel_delta"])
def test_a_far_token_reaches_through_the_state(tmp_path, kind, dtype):
    """States that forget slowly, and only one token that writes into them: it stands once, 250 to 300
    positions back - right before, on and right after a page border, and first of all - and reaches the
    last tokens only through the state carried from step to step.  Another token in its place changes
    their logits wholly."""
    if kind == "retention":
        layer = nx.retention(3, 24, 12, (0.999, 0.9995, 1.0), 16)
    else:
        layer = nx.channel_delta(3, 1, 24, 12, 3, 6)
    vocab = 24 if kind == "retention" else 40
    config = nx.one_layer(layer, vocab=vocab, width=48, streams=2)
    state = nx.random_state(config, 51, slow_decay=True)
    target, stand_in = 5, 6
    only_the_target_writes(config, state, target, kind)
    page, n = 16, 300
    reqs = {}
    for place in (15, 16, 17, 0, 49):
        toks = [t if t != target else stand_in for t in nx.tokens(70 + place, n, vocab)]
        toks[place] = target
        reqs[f"t{place}"] = toks
    want = {rid: plain.forward(config, state, t) for rid, t in reqs.items()}
    other = list(reqs["t16"])
    other[16] = stand_in
    assert float(nx.position_errors(plain.forward(config, state, other)[-1:], want["t16"][-1:])) > 0.3
    folder = nx.write(str(tmp_path / "m"), config, state)
    # retention in bfloat16: the shrunk values are small differences of large products of a rounded input
    # (4 % off by construction, whatever computes them); the effect looked for is ten times that
    tol = nx.TOL[dtype] * (2 if (kind, dtype) == ("retention", "bfloat16") else 1)
    for cut in ("decode_tail", "portions", "mixed"):
        schedule = CUTS[cut](reqs)
        engine = nx.make_engine(folder, dtype, page, rd.peak_tokens(schedule, page), poison=True)
        nx.compare(run_engine(engine, reqs, schedule), want, tol, f"far token, {kind}, {cut} [{dtype}]")


# ------------------------------------------------- long prompts at sizes between tiny and real
LONG = nx.model(640, 256, 2, 1e-5, [
    nx.latent(4, 32, 32, 64, 96, 96, 200, base=40000.0, mlp=nx.dense(512, 2.0)),
    nx.channel_delta(4, 2, 64, 32, 4, 32, nx.moe(16, 4, 64, 4, 2, scale=2.5), gate_rank=16),
    nx.retention(4, 32, 64, (0.9, 0.99, 0.999, 0.9995), 16, base=1e6, mlp=nx.dense(384, 1.5)),
    nx.latent(2, 48, 16, 64, 64, 48, 64, base=500.0, mlp=nx.moe(8, 2, 96, 2, 1)),
    nx.channel_delta(2, 2, 32, 64, 3, 24),
])


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_long_prompts(tmp_path, dtype):
    """Prompts of up to 1,500 tokens (two dozen pages of 64, windows of 200 and 64 that pass many of
    them, cached rows of 128 and 64 values on the tensor-core kernels in bfloat16, states that forget
    slowly), whole and in a mixed batch whose decoded tokens read hundreds of keys."""
    state = nx.random_state(LONG, 7, slow_decay=True)
    folder = nx.write(str(tmp_path / "m"), LONG, state)
    reqs = {f"r{i}": nx.tokens(11 * i + 3, n, LONG["vocab"]) for i, n in enumerate([1500, 700, 64, 65, 129])}
    for cut in ("whole", "mixed"):
        run_and_compare(folder, LONG, state, reqs, CUTS[cut](reqs), dtype, 64, f"long {cut}")


# --------------------------------------------------------- first tokens, long decoding
@pytest.mark.parametrize("dtype", list(DTYPES))
def test_first_tokens_and_long_decoding(models, dtype):
    """A request that starts with a single token and is decoded one token at a time for 200 steps (windows
    pass, pages go back, decode steps are replayed from a graph in bfloat16), beside a second request
    that joins later two tokens a step; against the whole sequences."""
    from freetoken_b200.engine import StepEntry
    config = nx.NX["A"]
    state = nx.random_state(config, nx.SEEDS["A"])
    a, b = nx.tokens(5, 201, config["vocab"]), nx.tokens(6, 120, config["vocab"])
    engine = nx.make_engine(models["A"], dtype, 4, 204 + 120)
    got_a, got_b = [], []
    routed = nx.routed_layers(config)
    ids_a, ids_b = [], []
    for i in range(len(a)):
        entries = [StepEntry("a", [a[i]], [0])]
        j = i - 60
        if 0 <= j < len(b) // 2:
            entries.append(StepEntry("b", b[2 * j:2 * j + 2], [0, 1]))
        probe = {"router_ids": []}
        logits = engine.step(entries, probe=probe).float().cpu()
        got_a.append(logits[0])
        got_b.extend(logits[1:])
        ids_a.append([x[0].cpu().long() for x in probe["router_ids"]])
        if len(entries) > 1:
            ids_b.extend([x[r].cpu().long() for x in probe["router_ids"]] for r in (1, 2))
    assert len(routed) == len(ids_a[0])
    want = {}
    for rid, toks, ids in (("a", a, ids_a), ("b", b, ids_b)):
        chosen = {layer: torch.stack([step[j] for step in ids]) for j, layer in enumerate(routed)}
        want[rid] = plain.forward(config, state, toks, expert_ids=chosen if dtype == "bfloat16" else None)
    nx.compare({"a": torch.stack(got_a), "b": torch.stack(got_b)}, want, nx.TOL[dtype], f"long decoding [{dtype}]")


# ------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("which", ["A", "B"])
def test_greedy_generation_through_the_scheduler(models, which, dtype):
    """``LLM.generate`` (scheduler, overlapped steps, graph replay of decode steps in bfloat16): every
    generated token is the plain model's own greedy choice for the sequence so far, unless its two best
    logits - or two router scores somewhere in the sequence - lie within rounding of each other."""
    from freetoken_b200 import LLM, SamplingParams
    config = nx.NX[which]
    state = nx.random_state(config, nx.SEEDS[which])
    llm = LLM(models[which], dtype, page_size=nx.PAGE[which], num_token_override=1024, max_running_req=3,
              max_extend_tokens=24)
    prompts = [nx.tokens(70 + i, n, config["vocab"]) for i, n in enumerate((3, 30, 11, 1, 47))]
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    tie = 1e-4 if dtype == "float32" else 8e-2
    route_tie = 5e-2
    ties = 0
    for prompt, result in zip(prompts, out):
        seq = list(prompt)
        assert len(result["token_ids"]) == 12
        for token in result["token_ids"]:
            margins = []
            logits = plain.forward(config, state, seq, margins=margins)[-1]
            if token != int(logits.argmax()):
                margin = min((float(m.min()) for m in margins), default=float("inf"))
                near = float(logits.max() - logits[token]) < tie or (dtype == "bfloat16" and margin < route_tie)
                assert near, (dtype, len(seq), token, int(logits.argmax()), float(logits.max() - logits[token]), margin)
                ties += 1
                if margin < route_tie:
                    break            # another expert somewhere in the sequence: what follows is another sequence
            seq.append(int(token))
    assert ties == 0 if dtype == "float32" else ties <= 4
    if dtype == "bfloat16":
        assert llm.engine.graph_replays > 0


# -------------------------------------------------------------------- the replay tool
def test_trace_replay_tool(models, tmp_path):
    """``bin/trace_run`` on a Nirelix folder (whose config.json does not state the width of the delta
    rule's two-step projections): a mixed schedule with exactly the pages its peak needs."""
    which = "C"
    reqs = requests_of(which)
    state = nx.random_state(nx.NX[which], nx.SEEDS[which])
    schedule = rd.mixed(reqs)
    page = nx.PAGE[which]
    got = rd.run_trace_tool(models[which], "float32", reqs, schedule, str(tmp_path / "out"),
                            rd.peak_tokens(schedule, page), page, nx.NX[which]["vocab"])
    nx.compare(got, expected_for(nx.NX[which], state, reqs, "float32"), nx.TOL["float32"], "trace_run, mixed")
