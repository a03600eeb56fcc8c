"""Position encodings a mixer applies to queries and keys.

Rotary: ``inv_freq_i = theta^(-2i/R)``, ``cos_sin[p] = [cos(p*inv_freq) |
sin(p*inv_freq)]`` in float32 over the first ``R = rotary_dim`` dims of every
head, the rest untouched (python/freetoken/layers/rotary.py:40-59).  Pairing is
NeoX halves ``(i, i+R/2)`` or interleaved ``(2i, 2i+1)``
(python/freetoken/kernel/triton/rope.py:62-78).  The table is computed on the
host in float32, as the reference computes it, and cut to the positions the
engine can reach.  ``none`` rotates nothing.

Two rules that stretch the frequencies for contexts longer than the one a model was trained on
(``scaling``, a dictionary with ``kind`` and the rule's constants; the reference's models use
neither):

* ``yarn``: with ``dim(t) = R ln(original / (2 pi t)) / (2 ln theta)``, ``lo = max(floor(dim(fast)),
  0)``, ``hi = min(ceil(dim(slow)), R - 1)`` and ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0,
  1)`` the frequency of pair ``i`` is ``f_i / factor * ramp_i + f_i (1 - ramp_i)``, and cosines and
  sines are multiplied by ``0.1 ln(factor) + 1``;
* ``llama3``: with the wavelength ``l = 2 pi / f``, ``f`` stays where ``l < original / high``, becomes
  ``f / factor`` where ``l > original / low``, and ``(1 - s) f / factor + s f`` with ``s = (original / l -
  low) / (high - low)`` in between.
"""

from __future__ import annotations

import math
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from .base import Position, register_position

# One cos|sin table per (rotary_dim, theta, device), shared by every layer that
# rotates the same way (the reference shares one module through a cached
# ``get_rope``, python/freetoken/layers/rotary.py:212-213).  A table only grows.
_TABLES: Dict[Tuple, torch.Tensor] = {}

SCALING_KINDS = ("yarn", "llama3")


def scaled_frequencies(rotary_dim: int, theta: float, scaling: Mapping[str, Any]) -> Tuple[torch.Tensor, float]:
    """``(frequencies [rotary_dim / 2] float64, factor on cosines and sines)`` under a scaling rule
    (the module's docstring states both rules)."""
    r, kind = int(rotary_dim), scaling.get("kind")
    f = float(theta) ** (-torch.arange(0, r, 2, dtype=torch.float64) / r)
    factor, original = float(scaling["factor"]), float(scaling["original"])
    if kind == "yarn":
        def dim_of(turns: float) -> float:
            return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))
        lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(dim_of(float(scaling["slow"]))), r - 1)
        ramp = ((torch.arange(r // 2, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0
    if kind == "llama3":
        low, high = float(scaling["low"]), float(scaling["high"])
        wavelength = 2.0 * math.pi / f
        # high == low leaves no wavelength between the two bounds: the blend is then never chosen
        s = (original / wavelength - low) / (high - low if high != low else 1.0)
        blended = (1.0 - s) * f / factor + s * f
        out = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blended))
        return out, 1.0
    raise ValueError(f"rotary scaling kind {kind!r} is not one of {list(SCALING_KINDS)}")


def rotary_table(rotary_dim: int, theta: float, device, positions: int, exact_angles: bool = False,
                 scaling: Optional[Mapping[str, Any]] = None) -> torch.Tensor:
    """``[>= positions, rotary_dim]`` float32 on ``device``: ``cos | sin`` of
    ``position * theta^(-2i/rotary_dim)``, computed on the host in float32; with
    ``exact_angles`` the angle, its cosine and sine are computed in float64 and rounded once,
    so that the float32 product ``position * frequency`` (half a unit in the last place of the
    angle, 3e-5 rad at position 1,000) does not enter.  With ``scaling`` the frequencies (and the
    size of cosines and sines) follow that rule, always with exact angles."""
    frozen = tuple(sorted((k, v) for k, v in scaling.items())) if scaling else None
    key = (int(rotary_dim), float(theta), torch.device(device), bool(exact_angles), frozen)
    table = _TABLES.get(key)
    if table is None or table.shape[0] < positions:
        r = int(rotary_dim)
        real = torch.float64 if (exact_angles or scaling) else torch.float
        magnitude = 1.0
        if scaling:
            inv_freq, magnitude = scaled_frequencies(r, theta, scaling)
        else:
            inv_freq = 1.0 / (float(theta) ** (torch.arange(0, r, 2, dtype=real) / r))
        t = torch.arange(positions, dtype=real)
        freqs = torch.einsum("i,j -> ij", t, inv_freq)
        table = (torch.cat((freqs.cos(), freqs.sin()), dim=-1) * magnitude).float().contiguous().to(device)
        _TABLES[key] = table
    return table


class _Rotary(Position):
    graph_capturable = True
    interleaved = False

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.max_position = int(spec.params["max_position"])
        self.exact_angles = bool(spec.params.get("exact_angles", False))
        # {"kind": "yarn", factor, original, fast, slow} or {"kind": "llama3", factor, original, low, high}
        self.scaling = dict(spec.params["scaling"]) if spec.params.get("scaling") else None
        if self.scaling and self.scaling.get("kind") not in SCALING_KINDS:
            raise ValueError(f"rotary scaling kind {self.scaling.get('kind')!r} is not one of {list(SCALING_KINDS)}")
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")

    def table(self, device, positions: int) -> Optional[torch.Tensor]:
        """``[>= positions, rotary_dim]`` float32 on ``device`` (``None`` when
        nothing rotates); every layer with the same rotation gets the same tensor."""
        if self.rotary_dim == 0:
            return None
        return rotary_table(self.rotary_dim, self.theta, device, min(positions, self.max_position),
                            self.exact_angles, self.scaling)


@register_position("rotary_neox")
class RotaryNeox(_Rotary):
    interleaved = False


@register_position("rotary_interleaved")
class RotaryInterleaved(_Rotary):
    interleaved = True


@register_position("none")
class NoPosition(Position):
    graph_capturable = True
    interleaved = False
    rotary_dim = 0

    def table(self, device, positions: int):
        return None
