"""A plain, slow implementation of the Nirelix decoder: one function per mechanism.

Everything is a loop or a dense tensor expression over one whole sequence in the working
precision of the weights handed in (the tests use float64); there is no cache, no state object
and no batching, and nothing here is shared with the engine's code.  ``cfg`` is the config.json
dictionary, ``w`` a dictionary of tensors by checkpoint name.

* streams: ``s`` copies of the residual; a sublayer reads ``sum_s in[s] x_s`` (layer-normed) and
  every stream becomes ``sum_s mix[s, t] x_s + out[t] y``.
* mixers: ``retention`` (a decaying outer-product state per head, rotated q and k),
  ``channel_delta`` (the gated delta rule with a decay per key channel), ``latent_attention``
  (keys and values made from a cached latent, one rotated key part shared by the heads, a
  sliding window).
* feed-forwards: dense with a clamped gate/up pair, or experts chosen inside the best groups.
"""

import math

import torch


# ------------------------------------------------------------------ small functions
def rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def layer_norm(v, weight, bias, eps):
    mean = v.mean(-1, keepdim=True)
    var = ((v - mean) ** 2).mean(-1, keepdim=True)
    return (v - mean) / torch.sqrt(var + eps) * weight + bias


def silu(v):
    return v * torch.sigmoid(v)


def softplus(v):
    return torch.where(v > 30, v, torch.log1p(torch.exp(torch.clamp(v, max=30.0))))


def angles(T, base, dims, first=0):
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.arange(first, first + T, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]


def rotate_halves(v, base, dims, first=0):
    """``v`` ``[T, heads, dim]``: dimension i of the first ``dims`` turns with i + dims/2."""
    a = angles(v.shape[0], base, dims, first)
    cos, sin = a.cos().to(v.dtype)[:, None, :], a.sin().to(v.dtype)[:, None, :]
    half = dims // 2
    x, y = v[..., :half], v[..., half:dims]
    return torch.cat([x * cos - y * sin, y * cos + x * sin, v[..., dims:]], dim=-1)


def rotate_pairs(v, base, dims, first=0):
    """``v`` ``[T, heads, dim]``: dimension 2i of the first ``dims`` turns with 2i + 1."""
    a = angles(v.shape[0], base, dims, first)
    cos, sin = a.cos().to(v.dtype)[:, None, :], a.sin().to(v.dtype)[:, None, :]
    x, y = v[..., 0:dims:2], v[..., 1:dims:2]
    turned = torch.stack([x * cos - y * sin, y * cos + x * sin], dim=-1).flatten(-2)
    return torch.cat([turned, v[..., dims:]], dim=-1)


def causal_conv(u, weight):
    """``u`` ``[T, C]``, ``weight`` ``[C, taps]`` whose last column weighs the current token."""
    T, C = u.shape
    taps = weight.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += weight[:, j] * u[src]
    return out


# ------------------------------------------------------------------------- mixers
def retention(h, w, p, m, eps):
    """Per head ``S <- decay S + k v^T``, ``o = S^T q``; ``o`` divided by its root mean square,
    gated by silu, projected."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    q = rotate_halves(q, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_halves(k, m["rot"]["base"], m["rot"]["dims"]) * D ** -0.5
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    out = rms(out, eps).reshape(T, H * V) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def channel_delta(h, w, p, m, eps):
    """The gated delta rule whose decay differs per key channel."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                    # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]                # [T, H * D]
    g = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * softplus(a).view(T, H, D))
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = g[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(T, H, V)
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(T, H * V) @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Softmax attention inside a window; queries through a normed latent, keys and values from
    a normed latent plus one rotated key part that all heads share."""
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(down[:, rank:].reshape(T, 1, R), m["rot"]["base"], m["rot"]["dims"])
    q_rot = rotate_pairs(q[..., D:], m["rot"]["base"], m["rot"]["dims"])
    k = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :D], k)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < m["mask"]["size"])
    scores = scores.masked_fill(~seen[None], float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(T, H * V)
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


MIXERS = {"retention": retention, "channel_delta": channel_delta, "latent_attention": latent_attention}


# ------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, p, mlp):
    limit = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def choose_experts(h, w, p, router, margins=None):
    """``(ids [T, top], weights [T, top])``: the largest choice scores inside the best groups.
    ``margins`` (a list) receives, per token, by how much the last chosen expert beat the first one
    left out, and the last kept group the first one dropped."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    per = E // groups["count"]
    grouped = choice.view(-1, groups["count"], per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = group_score.topk(groups["keep"], dim=-1).indices
    allowed = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
    allowed = allowed[:, :, None].expand(-1, -1, per).reshape(-1, E)
    masked = choice.masked_fill(~allowed, float("-inf"))
    ids = masked.topk(top, dim=-1).indices
    if margins is not None:
        m = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
        if top < E:
            best = masked.topk(top + 1, dim=-1).values
            m = torch.minimum(m, best[:, top - 1] - best[:, top])
        if groups["keep"] < groups["count"]:
            best = group_score.topk(groups["keep"] + 1, dim=-1).values
            m = torch.minimum(m, best[:, -2] - best[:, -1])
        margins.append(m)
    picked = s.gather(1, ids)
    return ids, picked / (picked.sum(-1, keepdim=True) + 1e-20) * router["scale"]


def expert_ff(h, w, p, mlp, ids=None, margins=None):
    """``ids`` (``[T, top]``) overrides the choice; the weights are always those of the scores."""
    router = mlp["router"]
    own_ids, weights = choose_experts(h, w, p, router, margins)
    if ids is not None:
        s = torch.sigmoid(h @ w[p + "router"].T).gather(1, ids)
        weights = s / (s.sum(-1, keepdim=True) + 1e-20) * router["scale"]
    else:
        ids = own_ids
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for slot in range(ids.shape[1]):
            e = f"{p}e{int(ids[t, slot])}."
            mid = silu(w[e + "gate"] @ h[t]) * (w[e + "up"] @ h[t])
            out[t] += weights[t, slot] * (w[e + "down"] @ mid)
    return out


# --------------------------------------------------------------------------- model
def sublayer(streams, w, prefix, q, fn, eps):
    """One hyper-connected sublayer on ``streams`` ``[s, T, W]``."""
    hc = f"{prefix}hc{q}."
    u = torch.einsum("s,stw->tw", w[hc + "in"], streams)
    y = fn(layer_norm(u, w[f"{prefix}norm{q}"], w[f"{prefix}norm{q}.b"], eps))
    return torch.einsum("sr,stw->rtw", w[hc + "mix"], streams) + w[hc + "out"][:, None, None] * y[None]


def forward(cfg, w, tokens, expert_ids=None, trace=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence.  ``expert_ids``: ``{layer: ids [T, top]}`` to use
    instead of the plain choice; ``trace``: a list that receives the sum of the streams after
    every layer; ``margins``: a list that receives every routed layer's choice margins."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = x[None].repeat(cfg.get("streams", 1), 1, 1)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mix = MIXERS[layer["type"]]
        streams = sublayer(streams, w, p, 1, lambda h: mix(h, w, p + "mix.", layer["mixer"], eps), eps)
        mlp = layer.get("mlp")
        if mlp:
            if mlp.get("kind", "dense") == "dense":
                ff = lambda h: dense_ff(h, w, p + "mlp.", mlp)
            else:
                ff = lambda h: expert_ff(h, w, p + "mlp.", mlp, None if expert_ids is None else expert_ids.get(i), margins)
            streams = sublayer(streams, w, p, 2, ff, eps)
        if trace is not None:
            trace.append(streams.sum(0))
    x = layer_norm(streams.sum(0), w["final.norm"], w["final.norm.b"], eps)
    return x @ w["head"].T


def expected_tensors(cfg):
    """``{name: shape}`` of a checkpoint of ``cfg``."""
    W, s = cfg["width"], cfg.get("streams", 1)
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "final.norm.b": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        has = [1] + ([2] if layer.get("mlp") else [])
        for q in has:
            out.update({f"{p}norm{q}": (W,), f"{p}norm{q}.b": (W,), f"{p}hc{q}.in": (s,), f"{p}hc{q}.out": (s,),
                        f"{p}hc{q}.mix": (s, s)})
        x = p + "mix."
        if layer["type"] == "retention":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out.update({x + "q": (H * D, W), x + "k": (H * D, W), x + "v": (H * V, W), x + "g": (H * V, W),
                        x + "o": (W, H * V)})
        elif layer["type"] == "channel_delta":
            H, G, D, V, taps, low = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], m["low_rank"]
            glow = m.get("gate_rank") or low
            # (low_rank, gate_rank: sizes a checkpoint states only through its tensor shapes; the tests'
            # configurations carry them so that weights can be made, the files' config.json does not)
            out.update({x + "q": (G * D, W), x + "k": (G * D, W), x + "v": (H * V, W),
                        x + "q.conv": (G * D, taps), x + "k.conv": (G * D, taps), x + "v.conv": (H * V, taps),
                        x + "b": (H, W), x + "A_log": (H,), x + "norm": (V,), x + "a1": (low, W),
                        x + "a2": (H * D, low), x + "dt_bias": (H * D,), x + "g1": (glow, W),
                        x + "g2": (H * V, glow), x + "o": (W, H * V)})
        else:
            H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            out.update({x + "dq": (m["q_rank"], W), x + "dq.norm": (m["q_rank"],),
                        x + "uq": (H * (D + R), m["q_rank"]), x + "dkv": (m["kv_rank"] + R, W),
                        x + "dkv.norm": (m["kv_rank"],), x + "uk": (H * D, m["kv_rank"]),
                        x + "uv": (H * V, m["kv_rank"]), x + "g": (H * V, W), x + "o": (W, H * V)})
        mlp = layer.get("mlp")
        f = p + "mlp."
        if mlp and mlp.get("kind", "dense") == "dense":
            out.update({f + "gate": (mlp["ff"], W), f + "up": (mlp["ff"], W), f + "down": (W, mlp["ff"])})
        elif mlp:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            out.update({f + "router": (E, W), f + "correction": (E,)})
            for e in range(E):
                out.update({f"{f}e{e}.gate": (ff, W), f"{f}e{e}.up": (ff, W), f"{f}e{e}.down": (W, ff)})
    return out
