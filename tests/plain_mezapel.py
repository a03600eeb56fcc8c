"""A plain, slow implementation of the Mezapel decoder: one function per mechanism.

Everything is a loop or a dense tensor expression over one whole sequence in the working
precision of the weights handed in (the tests use float64); there is no cache, no state object
and no batching, and nothing here is shared with the engine's code.  ``cfg`` is the config.json
dictionary, ``w`` a dictionary of tensors by checkpoint name.

* embedding: the token's row times a scale plus a row of a second table chosen by a hash of the
  token and the one before it (a row of its own for a sequence's first token);
* residual: a plain pre-norm sum, or ``streams`` copies joined by hyper-connections;
* mixers: ``attention`` (one norm over all of q and one over all of k, a rotated part with YaRN
  frequencies, a mask in chunks, softmax weights ``e^s / (1 + sum e^s)``, a gate per head) and
  ``attention_2`` (short convolutions behind the projections, a norm per head, Llama-3.1
  frequencies, capped scores, a sliding window, a learned sink per head, a gate per value);
* feed-forward: ``W_down (silu(W_gate h) (W_up h))``.
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


# ---------------------------------------------------------------------- embedding
def bigram_rows(tokens, big):
    """Row of the second table per token: a hash of (previous, current), the last row first."""
    buckets = int(big["buckets"])
    rows = []
    for t, tok in enumerate(tokens):
        if t == 0:
            rows.append(buckets)
        else:
            rows.append((int(tokens[t - 1]) * int(big["mul_prev"]) + int(tok) * int(big["mul_cur"])) % buckets)
    return rows


def embed(cfg, w, tokens):
    e = cfg.get("embedding") or {}
    ids = torch.tensor([int(t) for t in tokens], dtype=torch.long)
    x = w["embed"][ids] * float(e.get("scale", 1.0))
    if e.get("bigram"):
        x = x + w["bigram"][torch.tensor(bigram_rows(tokens, e["bigram"]), dtype=torch.long)]
    return x


# ------------------------------------------------------------------ rotation tables
def plain_frequencies(base, dims):
    return [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]


def yarn_frequencies(base, dims, s):
    """Frequencies blended between ``f`` and ``f / factor`` along a ramp over the pair index, and
    the factor on cosines and sines."""
    factor, original = float(s["factor"]), float(s["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(s["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(s["slow"]))), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def llama3_frequencies(base, dims, s):
    """Short wavelengths keep their frequency, long ones are divided by ``factor``, the ones
    between are blended."""
    factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    out = []
    for f in plain_frequencies(base, dims):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            # only reached with high > low: with equal bounds a wavelength is on one side or the other
            # (one that lies exactly on the bound is divided by the factor here)
            t = (original / wavelength - low) / (high - low) if high != low else 0.0
            out.append((1.0 - t) * f / factor + t * f)
    return out, 1.0


def rotation(rot, kind):
    """``(frequencies, magnitude)`` of a mixer's ``rot`` entry; ``kind`` names the scaling rule
    the mixer uses when the entry has a ``scaling`` part."""
    dims, base = int(rot["dims"]), float(rot["base"])
    if not rot.get("scaling"):
        return plain_frequencies(base, dims), 1.0
    return (yarn_frequencies if kind == "yarn" else llama3_frequencies)(base, dims, rot["scaling"])


def rotate_halves(v, freqs, magnitude, first=0):
    """``v`` ``[T, heads, dim]``: dimension i of the first ``2 len(freqs)`` turns with i + len(freqs)."""
    half = len(freqs)
    if half == 0:
        return v
    pos = torch.arange(first, first + v.shape[0], dtype=torch.float64)
    a = pos[:, None] * torch.tensor(freqs, dtype=torch.float64)[None, :]
    cos, sin = (a.cos() * magnitude).to(v.dtype)[:, None, :], (a.sin() * magnitude).to(v.dtype)[:, None, :]
    x, y = v[..., :half], v[..., half:2 * half]
    return torch.cat([x * cos - y * sin, y * cos + x * sin, v[..., 2 * half:]], dim=-1)


# ------------------------------------------------------------------------- mixers
def masked_softmax_with_sink(scores, visible, sink):
    """``scores`` ``[T, T]`` of one head; ``sink``: a score without key or value that takes part
    in the denominator only.  Returns the weights of the visible keys."""
    out = torch.zeros_like(scores)
    for i in range(scores.shape[0]):
        js = [j for j in range(scores.shape[1]) if visible(i, j)]
        s = scores[i, js]
        top = max(float(s.max()), float(sink))
        e = torch.exp(s - top)
        out[i, js] = e / (e.sum() + math.exp(float(sink) - top))
    return out


def attention(h, w, p, m, eps):
    """Mixer ``attention``: norm over all of q and all of k, part of each head rotated with YaRN
    frequencies, keys of the query's own chunk only, softmax weights ``e^s / (1 + sum e^s)``, a
    sigmoid gate per head."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).view(T, G, V)
    freqs, magnitude = rotation(m["rot"], "yarn")
    q = rotate_halves(q.view(T, H, D), freqs, magnitude)
    k = rotate_halves(k.view(T, G, D), freqs, magnitude)
    size = int(m["mask"]["size"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    heads = []
    for i in range(H):
        g = i // (H // G)
        scores = (q[:, i] @ k[:, g].T) * float(m["scale"])
        weights = masked_softmax_with_sink(scores, lambda a, b: b <= a and a // size == b // size, 0.0)
        heads.append((weights @ v[:, g]) * gate[:, i:i + 1])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def attention_2(h, w, p, m, eps):
    """Mixer ``attention_2``: q, k and v through short causal convolutions, q and k normed per
    head with a weight all heads share, every head dimension (or the first ``rot.dims``) rotated
    with Llama-3.1 frequencies, scores capped by tanh, a sliding window, a learned sink per head,
    a sigmoid gate per output value."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q = rms(q.view(T, H, D), eps) * w[p + "q.norm"]
    k = rms(k.view(T, G, D), eps) * w[p + "k.norm"]
    v = v.view(T, G, V)
    freqs, magnitude = rotation(m["rot"], "llama3")
    q, k = rotate_halves(q, freqs, magnitude), rotate_halves(k, freqs, magnitude)
    size = int(m["mask"]["size"])
    cap = float(m.get("softcap") or 0.0)
    heads = []
    for i in range(H):
        g = i // (H // G)
        scores = (q[:, i] @ k[:, g].T) * float(m["scale"])
        if cap:
            scores = cap * torch.tanh(scores / cap)
        weights = masked_softmax_with_sink(scores, lambda a, b: 0 <= a - b < size, float(w[p + "sink"][i]))
        heads.append(weights @ v[:, g])
    return (torch.cat(heads, dim=-1) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"attention": attention, "attention_2": attention_2}


def dense_ff(h, w, p, mlp):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ------------------------------------------------------------------- the whole model
def run_order(cfg):
    """Indices of the layers in the order they run: a looped range repeats as a whole."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def sublayer(streams, w, prefix, q, fn, eps):
    """One sublayer.  ``streams`` is a list of residual copies (hyper-connections) or a single
    tensor (plain pre-norm residual)."""
    if not isinstance(streams, list):
        return streams + fn(layer_norm(streams, w[f"{prefix}.norm{q}"], w[f"{prefix}.norm{q}.b"], eps))
    S = len(streams)
    w_in, w_out, w_mix = w[f"{prefix}.hc{q}.in"], w[f"{prefix}.hc{q}.out"], w[f"{prefix}.hc{q}.mix"]
    u = sum(w_in[s] * streams[s] for s in range(S))
    y = fn(layer_norm(u, w[f"{prefix}.norm{q}"], w[f"{prefix}.norm{q}.b"], eps))
    return [sum(w_mix[s, t] * streams[s] for s in range(S)) + w_out[t] * y for t in range(S)]


def forward(cfg, w, tokens, trace=None):
    """Logits ``[T, vocab]`` of one sequence.  ``trace``: a list that receives the residual (the
    sum of the streams) after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = embed(cfg, w, tokens)
    S = cfg.get("streams")
    streams = [x.clone() for _ in range(int(S))] if S else x
    for i in run_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}"
        mix = MIXERS[layer["type"]]
        streams = sublayer(streams, w, p, 1, lambda h: mix(h, w, p + ".mix.", layer["mixer"], eps), eps)
        if layer.get("mlp"):
            streams = sublayer(streams, w, p, 2, lambda h: dense_ff(h, w, p + ".mlp.", layer["mlp"]), eps)
        if trace is not None:
            trace.append(sum(streams) if isinstance(streams, list) else streams)
    x = sum(streams) if isinstance(streams, list) else streams
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T


def expected_tensors(cfg):
    """Name -> shape of every tensor a checkpoint of ``cfg`` holds."""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    out = {"embed": (V, W)}
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        out["bigram"] = (int(big["buckets"]) + 1, W)
    S = cfg.get("streams")
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, G, D, Vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        subs = [1] + ([2] if layer.get("mlp") else [])
        for q in subs:
            out[f"{p}norm{q}"] = (W,)
            out[f"{p}norm{q}.b"] = (W,)
            if S:
                out[f"{p}hc{q}.in"] = (int(S),)
                out[f"{p}hc{q}.out"] = (int(S),)
                out[f"{p}hc{q}.mix"] = (int(S), int(S))
        out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = (H * D, W), (G * D, W), (G * Vd, W)
        out[p + "mix.o"] = (W, H * Vd)
        if layer["type"] == "attention":
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = (H * D,), (G * D,)
            out[p + "mix.g"] = (H, W)
        else:
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = (D,), (D,)
            out[p + "mix.g"] = (H * Vd, W)
            out[p + "mix.sink"] = (H,)
            if m.get("conv"):
                taps = int(m["conv"])
                out[p + "mix.q.conv"], out[p + "mix.k.conv"], out[p + "mix.v.conv"] = (H * D, taps), (G * D, taps), (G * Vd, taps)
        if layer.get("mlp"):
            ff = int(layer["mlp"]["ff"])
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (ff, W), (ff, W), (W, ff)
    out["final.norm"], out["final.norm.b"], out["head"] = (W,), (W,), (V, W)
    return out
