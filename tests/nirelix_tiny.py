"""Tiny Nirelix configurations, random weights for them, and helpers of the tests.

The configurations differ from each other in every size and constant: widths, stream counts (one,
two, four), head counts, key sizes below, equal to and above value sizes, windows of 1, of a few
tokens, shorter and longer than a page, rotation of a part of a head and of all of it, latents
narrower and wider than the heads, groups of experts of one, two and four of which one, some or
all are kept, convolutions of 1 to 4 taps, two-step projections whose middles are equal or not, layers without feed-forward, every layer order.
"""

from __future__ import annotations

import copy
from typing import Dict, List

import torch

import plain_nirelix as plain
from fazinex_tiny import make_engine, position_errors, tokens, write_model  # noqa: F401  (re-exported)
from tonapel_tiny import compare  # noqa: F401  (re-exported)


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0, mlp=None):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                                           "rot": {"base": base, "dims": rot_dims}}, "mlp": mlp}


def channel_delta(heads, kv_heads, dim, vdim, conv, low_rank, mlp=None, gate_rank=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "low_rank": low_rank}
    if gate_rank:
        mixer["gate_rank"] = gate_rank
    return {"type": "channel_delta", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base=10000.0, scale=None, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                      "kv_rank": kv_rank, "scale": scale or (dim + rot_dim) ** -0.5, "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dim}}, "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, count, keep, scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


def model(vocab, width, streams, eps, layers):
    return {"architecture": "Nirelix", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps},
            "layers": layers}


# awkward sizes, nothing a multiple of 8; a window of 7 and of 1; two streams; a layer without feed-forward
NX_A: Dict = model(150, 40, 2, 1e-5, [
    channel_delta(4, 2, 12, 10, 2, 5, moe(6, 2, 24, 3, 2, scale=1.5), gate_rank=9),
    latent(3, 6, 4, 10, 14, 18, 7, base=100.0, mlp=dense(56, 0.8)),
    retention(3, 10, 6, (0.9, 0.97, 0.995), 6, base=300.0),
    latent(2, 12, 2, 5, 9, 20, 1, base=50.0, scale=0.4, mlp=moe(4, 3, 20, 1, 1)),
    retention(2, 20, 28, (0.5, 0.999), 20, mlp=dense(30, 3.0)),
])

# sizes the tensor-core attention kernels take (a cached row of 64 and of 128 values), pages of 64, windows
# shorter than, equal to and longer than a page; four streams
NX_B: Dict = model(320, 128, 4, 2e-6, [
    latent(4, 32, 32, 32, 48, 96, 100, mlp=dense(256, 2.0)),
    retention(4, 64, 32, (0.9, 0.99, 0.999, 0.96875), 32, base=500000.0, mlp=moe(8, 2, 64, 4, 2, scale=2.0)),
    latent(8, 16, 16, 64, 64, 48, 64, base=5000.0, mlp=moe(6, 1, 48, 6, 3)),
    channel_delta(4, 2, 64, 64, 4, 16, dense(192, 1.0)),
    latent(2, 64, 64, 32, 32, 64, 130, base=30000.0),
])

# one stream; recurrent layers first (no paged cache before the last layer); all groups kept; one expert
# of one; a width that is no multiple of 4 (no 16-byte pieces anywhere along a row of the residual)
NX_C: Dict = model(97, 70, 1, 1e-4, [
    retention(1, 33, 9, (0.98,), 0, mlp=moe(1, 1, 30, 1, 1, scale=0.7)),
    channel_delta(6, 6, 8, 12, 1, 3, dense(100, 0.5)),
    channel_delta(3, 1, 40, 36, 3, 24, moe(8, 4, 16, 2, 2), gate_rank=8),
    latent(6, 5, 8, 7, 11, 25, 33, base=1000.0),
])

NX = {"A": NX_A, "B": NX_B, "C": NX_C}
PAGE = {"A": 4, "B": 64, "C": 12}
SEEDS = {"A": 61, "B": 62, "C": 63}


def random_state(config: Dict, seed: int, slow_decay: bool = False) -> Dict[str, torch.Tensor]:
    """Every tensor of a model of ``config`` by name, drawn so that activations stay of order one and
    rounded to bfloat16 (what the file holds), as float64.  ``slow_decay``: delta-rule states that
    forget slowly, so that a token far back still counts."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    streams = config.get("streams", 1)
    for name, shape in plain.expected_tensors(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        std, mean, eye = (shape[-1] ** -0.5 if len(shape) > 1 else 1.0), 0.0, 0.0
        if leaf in ("norm1", "norm2", "final.norm", "mix.norm", "mix.dq.norm", "mix.dkv.norm"):
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
        elif leaf == "mix.A_log":
            std, mean = 0.5, -6.0 if slow_decay else -0.5
        elif leaf == "mix.dt_bias":
            std, mean = 0.5, -0.5
        elif leaf == "embed":
            std = 1.0
        elif leaf == "mlp.router":
            std = 2.0 * shape[-1] ** -0.5
        elif leaf == "mlp.correction":
            std = 0.2
        t = torch.randn(*shape, generator=g, dtype=torch.float64) * std + mean
        if eye:
            t = t + eye * torch.eye(shape[0], dtype=torch.float64)
        out[name] = t.to(torch.bfloat16).double()
    return out


def file_config(config: Dict) -> Dict:
    """``config`` as a checkpoint's config.json states it: without the sizes that only tensor shapes give."""
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        layer["mixer"].pop("low_rank", None)
        layer["mixer"].pop("gate_rank", None)
    return out


def as_file(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.to(torch.bfloat16) for k, v in state.items()}


def write(folder: str, config: Dict, state: Dict[str, torch.Tensor]) -> str:
    return write_model(folder, file_config(config), as_file(state))


def write_tiny(folder: str, which: str) -> str:
    return write(folder, NX[which], random_state(NX[which], SEEDS[which]))


def one_layer(layer: Dict, vocab=90, width=48, streams=3, eps=1e-6) -> Dict:
    return model(vocab, width, streams, eps, [copy.deepcopy(layer)])


def routed_layers(config: Dict) -> List[int]:
    return [i for i, l in enumerate(config["layers"]) if l["mlp"] and l["mlp"]["kind"] == "moe"]


# Largest allowed error of a position's logits (see fazinex_tiny.position_errors).  float32: summation
# orders differ, and recurrences carry their rounding along.  bfloat16: every stored activation is
# rounded to 8 bits; a lost state, a window one token off, a lost key or a stream mixed the wrong way
# round gives 0.2 and more.
TOL = {"float32": 5e-5, "bfloat16": 6e-2}
