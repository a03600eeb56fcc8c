"""Tiny Mezapel configurations, random weights for them, and helpers of the tests.

The configurations differ from each other in every size and constant: widths, stream counts (two,
four, one, and no ``streams`` key at all), head counts and groupings (one key head for all, one per
head), key sizes below, equal to and above value sizes, chunks and windows of 1, of a few tokens,
shorter and longer than a page, rotation of nothing, of a part and of all of a head, with and
without frequency scaling, convolutions of 2 to 4 taps and none, scores capped and not, an
embedding with and without the hashed second table, loops over the first layers, the middle,
everything and none, layers without feed-forward, every layer order.
"""

from __future__ import annotations

import copy
from typing import Dict

import torch

import plain_mezapel as plain
from fazinex_tiny import make_engine, position_errors, tokens, write_model  # noqa: F401  (re-exported)
from tonapel_tiny import compare  # noqa: F401  (re-exported)


def yarn(factor, original, fast=24.0, slow=1.5):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def llama3(factor, original, low=0.5, high=3.0):
    return {"factor": factor, "original": original, "low": low, "high": high}


def attention(heads, kv_heads, dim, vdim, chunk, rot_dims, base=10000.0, scaling=None, scale=None, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "mask": {"size": chunk}, "rot": rot, "scale": scale or dim ** -0.5},
            "mlp": mlp}


def attention_2(heads, kv_heads, dim, vdim, window, rot_dims, conv, softcap=None, base=10000.0, scaling=None,
                scale=None, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = scaling
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": rot,
             "scale": scale or dim ** -0.5}
    if conv:
        mixer["conv"] = conv
    if softcap:
        mixer["softcap"] = softcap
    return {"type": "attention_2", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def model(vocab, width, streams, eps, layers, scale=1.0, bigram=None, loop=None):
    out = {"architecture": "Mezapel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "layers": layers}
    if streams is not None:
        out["streams"] = streams
    if bigram:
        out["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# awkward sizes, nothing a multiple of 8; a chunk of 7 and of 1, a window of 5; two streams; a layer without
# feed-forward; value heads wider and narrower than key heads; the loop covers the middle
MZ_A: Dict = model(150, 40, 2, 1e-5, [
    attention(4, 2, 12, 10, 7, 6, base=100.0, scaling=yarn(4.0, 16), mlp=dense(56)),
    attention_2(3, 3, 10, 14, 5, 10, 2, softcap=5.0, base=300.0, scaling=llama3(7.0, 32, 1.0, 2.0), mlp=dense(24)),
    attention(2, 1, 6, 6, 1, 0),
    attention_2(6, 2, 14, 6, 9, 4, 4, scale=0.4, mlp=dense(30)),
], scale=3.0, bigram=(37, 11, 5), loop=(1, 3, 2))

# sizes the tensor-core attention kernels take (heads of 64 and 128 values), pages of 64, chunks and windows
# shorter than, equal to and longer than a page; four streams; the loop covers the first layer
MZ_B: Dict = model(320, 128, 4, 2e-6, [
    attention(4, 2, 64, 64, 100, 32, base=500000.0, scaling=yarn(5.0, 64), mlp=dense(256)),
    attention_2(8, 2, 128, 128, 64, 128, 4, softcap=20.0, base=3e6, scaling=llama3(6.0, 128), mlp=dense(192)),
    attention(2, 2, 128, 64, 64, 64, base=5000.0, scale=0.15),
    attention_2(4, 1, 64, 32, 130, 16, 3, base=30000.0, mlp=dense(128)),
    attention(8, 1, 32, 32, 33, 32, base=777.0, scaling=yarn(2.0, 40, fast=8.0, slow=2.0), mlp=dense(64)),
], scale=11.3, bigram=(1021, 31, 7), loop=(0, 1, 3))

# one stream with connection weights; no hashed table; no convolution in one layer; a width that is no
# multiple of 4; the loop covers everything
MZ_C: Dict = model(97, 70, 1, 1e-4, [
    attention_2(1, 1, 33, 9, 33, 32, 0, softcap=2.0),
    attention(6, 6, 8, 12, 33, 8, mlp=dense(100)),
    attention_2(3, 1, 40, 36, 2, 0, 3, mlp=dense(16)),
], scale=0.5, loop=(0, 3, 2))

# no ``streams`` key: the plain pre-norm residual; no loop; a hashed table of one bucket
MZ_D: Dict = model(60, 48, None, 1e-6, [
    attention(3, 1, 16, 16, 12, 8, scaling=yarn(16.0, 8), mlp=dense(40)),
    attention_2(2, 2, 24, 8, 6, 24, 2, softcap=50.0, scaling=llama3(2.0, 16, 0.5, 8.0), mlp=dense(72)),
], bigram=(1, 3, 3))

MZ = {"A": MZ_A, "B": MZ_B, "C": MZ_C, "D": MZ_D}
PAGE = {"A": 4, "B": 64, "C": 12, "D": 8}
SEEDS = {"A": 81, "B": 82, "C": 83, "D": 84}


def random_state(config: Dict, seed: int) -> Dict[str, torch.Tensor]:
    """Every tensor of a model of ``config`` by name, drawn so that activations stay of order one and
    rounded to bfloat16 (what the file holds), as float64.  Sinks are drawn around 3, so that a sink left
    out changes a head's output by a quarter."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    streams = config.get("streams") or 1
    scale = float(config["embedding"].get("scale", 1.0))
    for name, shape in plain.expected_tensors(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        std, mean, eye = (shape[-1] ** -0.5 if len(shape) > 1 else 1.0), 0.0, 0.0
        if leaf in ("norm1", "norm2", "final.norm", "mix.q.norm", "mix.k.norm"):
            std, mean = 0.2, 1.0
        elif leaf.endswith(".b") and len(shape) == 1:
            std = 0.2
        elif leaf.endswith(".in"):
            std, mean = 0.2 / streams, 1.0 / streams
        elif leaf.endswith(".out"):
            std, mean = 0.2, 1.0
        elif leaf.endswith(".mix") and len(shape) == 2 and "hc" in leaf:
            std, eye = 0.2 / streams, 1.0
        elif leaf.endswith(".conv"):
            std = 0.5
        elif leaf == "mix.sink":
            std, mean = 1.0, 3.0
        elif leaf == "embed":
            std = 1.0 / scale
        elif leaf == "bigram":
            std = 0.7
        t = torch.randn(*shape, generator=g, dtype=torch.float64) * std + mean
        if eye:
            t = t + eye * torch.eye(shape[0], dtype=torch.float64)
        out[name] = t.to(torch.bfloat16).double()
    return out


def as_file(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.to(torch.bfloat16) for k, v in state.items()}


def write(folder: str, config: Dict, state: Dict[str, torch.Tensor]) -> str:
    return write_model(folder, copy.deepcopy(config), as_file(state))


def write_tiny(folder: str, which: str) -> str:
    return write(folder, MZ[which], random_state(MZ[which], SEEDS[which]))


def one_layer(layer: Dict, vocab=90, width=48, streams=3, eps=1e-6, scale=2.0, bigram=(23, 7, 3)) -> Dict:
    return model(vocab, width, streams, eps, [copy.deepcopy(layer)], scale=scale, bigram=bigram)


# Largest allowed error of a position's logits (see fazinex_tiny.position_errors).  float32: summation
# orders differ.  bfloat16: every stored activation is rounded to 8 bits; a window or a chunk one token
# off, a lost key, a sink left out or a stream mixed the wrong way round gives 0.2 and more.
TOL = {"float32": 5e-5, "bfloat16": 6e-2}
