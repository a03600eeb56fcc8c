"""Mixers that carry a state of fixed size per request instead of a cache that grows.

Both start with one merged input projection and a short causal convolution over
time (per channel, SiLU behind it) whose last ``taps - 1`` inputs are part of the
request's state, run a recurrence per head in float32, gate and RMS-norm the
read-out and end with an output projection.  In this file's notation ``S`` is a
head's state, ``x``/``v`` its input row of ``head_dim`` values:

* ``ssd`` (the recurrence of Mamba-2): ``step = softplus(dt + dt_bias)``,
  ``S <- exp(-exp(A) step) S + step B x^T``, ``y = S^T C + D x`` with ``B``, ``C``
  of ``state_dim`` values shared by the heads of a group; ``y * silu(z)`` is
  RMS-normed in ``norm_groups`` parts of the row.
* ``gated_delta`` (the gated delta rule): q and k unit vectors, ``g = exp(-exp(A)
  softplus(a + dt_bias))``, ``b = sigmoid(beta)``; ``S <- g S``, ``u = b (v - S^T k)``,
  ``S <- S + k u^T``, ``o = S^T q``; each head's ``o`` is RMS-normed, then gated by
  ``silu(gate)``.

* ``channel_delta``: the same rule with a decay per key channel, ``g_n = exp(-exp(A_h)
  softplus(a_n + dt_bias_n))`` with ``a = W_a2 (W_a1 h)`` through a narrow middle, acting on the
  rows of ``S``; the read-out's gate is ``sigmoid(W_g2 (W_g1 h))``.
* ``retention``: ``S <- c_h S + k v^T``, ``o = S^T q`` with a constant ``c_h`` per head, q and k
  rotated by their position, no convolution; ``o`` is RMS-normed per head without a weight and
  gated by ``silu``.

A request's state is one float32 row ``[convolution inputs | recurrent state]`` in
its slot (:class:`StateNeed`); the kernels take segments of any length, so a
prompt portion and a decoded token run the same code.  The reference keeps such
state in per-request slots too (python/freetoken/kvcache/linear_state_pool.py:32-78).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from ..weights.spec import Cat, Init, Name, TensorSpec
from . import linear
from .base import POSITIONS, CacheView, Mixer, StepContext, register_mixer


class _Recurrent(Mixer):
    graph_capturable = True
    writes_into_out = True

    conv_channels: int
    taps: int
    state_values: int

    def cache_need(self):
        return StateNeed(((self.taps - 1) * self.conv_channels + self.state_values,), "float32")

    def _states(self, cache: CacheView):
        """``(convolution inputs, recurrent state)`` as column ranges of the slots' rows."""
        if cache.state is None or not cache.writes:
            raise ValueError(f"{type(self).__name__} needs state slots of its own")
        cut = (self.taps - 1) * self.conv_channels
        return cache.state[:, :cut], cache.state[:, cut:]

    def libraries(self, dtype) -> List[str]:
        return ["recurrent"] + linear.libraries(dtype)


@register_mixer("ssd")
class SelectiveStateSpace(_Recurrent):
    """params: ``hidden_size, heads, head_dim, state_dim, groups, conv_taps, norm_groups,
    norm_eps``, ``scope`` and ``names`` (in, conv, conv_bias, dt_bias, a_log, d, norm, o below
    the scope).  The input projection's rows are ``z | x | B | C | dt``."""

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.P = int(p["head_dim"])
        self.N = int(p["state_dim"])
        self.G = int(p["groups"])
        self.taps = int(p["conv_taps"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.eps = float(p["norm_eps"])
        self.inner = self.heads * self.P
        if self.heads % self.G or self.inner % self.norm_groups or self.taps < 1 or self.N > 256:
            raise ValueError("ssd: heads must be a multiple of groups, the row a multiple of norm_groups, "
                             "state_dim at most 256")
        self.conv_channels = self.inner + 2 * self.G * self.N
        self.state_values = self.heads * self.N * self.P
        scope = self.name(p["scope"])
        self.names = {key: f"{scope}.{local}" for key, local in p["names"].items()}
        self.w: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> List[TensorSpec]:
        n, C = self.names, self.conv_channels
        small = dict(role="small32", tag="recurrent")
        return [
            TensorSpec(n["in"], (self.inner + C + self.heads, self.hidden)),
            TensorSpec(n["conv"], (C, self.taps), init=Init(0.0, 0.3), **small),
            TensorSpec(n["conv_bias"], (C,), init=Init(0.0, 0.1), **small),
            TensorSpec(n["dt_bias"], (self.heads,), init=Init(-1.0, 0.5), **small),
            TensorSpec(n["a_log"], (self.heads,), init=Init(-1.0, 0.5), **small),
            TensorSpec(n["d"], (self.heads,), init=Init(1.0, 0.2), **small),
            TensorSpec(n["norm"], (self.inner,), role="small32", init=Init(1.0, 0.0), tag="norm"),
            TensorSpec(n["o"], (self.hidden, self.inner), tag="residual_out"),
        ]

    def bind(self, tensors, dtype) -> None:
        self.w = {key: tensors[name] for key, name in self.names.items()}

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T, ws, w = x.shape[0], ctx.workspace, self.w
        inner, C = self.inner, self.conv_channels
        conv_state, state = self._states(cache)
        proj = linear.linear(x, w["in"], ws.get("ssd.in", (T, inner + C + self.heads), ctx.dtype))
        xbc = ws.get("ssd.xbc", (T, C), ctx.dtype)
        ops.conv_silu(proj[:, inner:inner + C], xbc, w["conv"], w["conv_bias"], conv_state, ctx.token_seg,
                      ctx.seg_slot, ctx.seg_q_start)
        y = ws.get("ssd.y", (T, inner), torch.float32)
        ops.ssd_scan(xbc, proj[:, inner + C:], w["dt_bias"], w["a_log"], w["d"], state, y, ctx.seg_slot,
                     ctx.seg_q_start, self.heads, self.P, self.N, self.G)
        gated = ws.get("ssd.gated", (T, inner), ctx.dtype)
        ops.gated_norm(y, proj[:, :inner], w["norm"], gated, self.norm_groups, self.eps, gate_first=True)
        if out is None:
            out = ws.get("ssd.out", (T, self.hidden), ctx.dtype)
        return linear.linear(gated, w["o"], out)


@register_mixer("gated_delta")
class GatedDelta(_Recurrent):
    """params: ``hidden_size, heads, key_heads, key_dim, head_dim, conv_taps, norm_eps, unit_eps``
    (under the root of the unit norms; default 1e-6), ``scope`` and ``names`` (q, k, v, gate,
    beta, decay: the projections; q_conv, k_conv, v_conv; a_log, dt_bias, norm, o; in and conv:
    the merged projection and convolution the model keeps).  Query / key head ``h // (heads /
    key_heads)`` serves head ``h``; q is multiplied by ``key_dim ** -0.5`` after its unit norm."""

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.G = int(p["key_heads"])
        self.D = int(p["key_dim"])
        self.P = int(p["head_dim"])
        self.taps = int(p["conv_taps"])
        self.eps = float(p["norm_eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        if self.heads % self.G or self.taps < 1 or self.D > 256:
            raise ValueError("gated_delta: heads must be a multiple of key_heads, key_dim at most 256")
        self.inner = self.heads * self.P
        self.conv_channels = 2 * self.G * self.D + self.inner
        self.state_values = self.heads * self.D * self.P
        scope = self.name(p["scope"])
        self.names = {key: f"{scope}.{local}" for key, local in p["names"].items()}
        self.w: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden
        kd = self.G * self.D
        small = dict(role="small32", tag="recurrent")
        rows = (("q", kd), ("k", kd), ("v", self.inner), ("gate", self.inner), ("beta", self.heads),
                ("decay", self.heads))
        convs = (("q_conv", kd), ("k_conv", kd), ("v_conv", self.inner))
        return [
            TensorSpec(n["in"], (sum(r for _, r in rows), H),
                       sources=(Cat(tuple(Name(n[key], (r, H)) for key, r in rows), 0),)),
            TensorSpec(n["conv"], (self.conv_channels, self.taps), init=Init(0.0, 0.3),
                       sources=(Cat(tuple(Name(n[key], (r, self.taps)) for key, r in convs), 0),), **small),
            TensorSpec(n["a_log"], (self.heads,), init=Init(-1.0, 0.5), **small),
            TensorSpec(n["dt_bias"], (self.heads,), init=Init(-1.0, 0.5), **small),
            TensorSpec(n["norm"], (self.P,), role="small32", init=Init(1.0, 0.0), tag="norm"),
            TensorSpec(n["o"], (H, self.inner), tag="residual_out"),
        ]

    def bind(self, tensors, dtype) -> None:
        self.w = {key: tensors[self.names[key]] for key in ("in", "conv", "a_log", "dt_bias", "norm", "o")}

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T, ws, w = x.shape[0], ctx.workspace, self.w
        C, inner, heads = self.conv_channels, self.inner, self.heads
        conv_state, state = self._states(cache)
        proj = linear.linear(x, w["in"], ws.get("delta.in", (T, C + inner + 2 * heads), ctx.dtype))
        qkv = ws.get("delta.qkv", (T, C), ctx.dtype)
        ops.conv_silu(proj[:, :C], qkv, w["conv"], None, conv_state, ctx.token_seg, ctx.seg_slot,
                      ctx.seg_q_start)
        o = ws.get("delta.o", (T, inner), torch.float32)
        gates = C + inner
        ops.delta_scan(qkv, proj[:, gates:gates + heads], proj[:, gates + heads:], w["dt_bias"], w["a_log"],
                       state, o, ctx.seg_slot, ctx.seg_q_start, heads, self.G, self.D, self.P, self.unit_eps,
                       self.D ** -0.5)
        gated = ws.get("delta.gated", (T, inner), ctx.dtype)
        ops.gated_norm(o, proj[:, C:C + inner], w["norm"], gated, heads, self.eps, gate_first=False)
        if out is None:
            out = ws.get("delta.out", (T, self.hidden), ctx.dtype)
        return linear.linear(gated, w["o"], out)


@register_mixer("channel_delta")
class ChannelDelta(_Recurrent):
    """params: ``hidden_size, heads, key_heads, key_dim, head_dim, conv_taps, low_rank`` (the width of
    the middle of the decay's two-step projection), ``gate_rank`` (the same of the gate's; default:
    ``low_rank``), ``norm_eps, unit_eps``, ``scope``
    and ``names`` (q, k, v, beta: projections; decay_down, decay_up, gate_down, gate_up: the two steps
    of the decay's and the gate's; q_conv, k_conv, v_conv; a_log, dt_bias, norm, o; in and conv: the
    merged projection and convolution the model keeps).  ``dt_bias`` has one entry per head and key
    channel, ``norm`` one per value of a head (shared by the heads)."""

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.G = int(p["key_heads"])
        self.D = int(p["key_dim"])
        self.P = int(p["head_dim"])
        self.taps = int(p["conv_taps"])
        self.low = int(p["low_rank"])
        self.gate_low = int(p.get("gate_rank") or self.low)
        self.eps = float(p["norm_eps"])
        self.unit_eps = float(p.get("unit_eps", 1e-6))
        if self.heads % self.G or self.taps < 1 or self.D > 256 or self.low < 1 or self.gate_low < 1:
            raise ValueError("channel_delta: heads must be a multiple of key_heads, key_dim at most 256")
        self.inner = self.heads * self.P
        self.conv_channels = 2 * self.G * self.D + self.inner
        self.state_values = self.heads * self.D * self.P
        scope = self.name(p["scope"])
        self.names = {key: f"{scope}.{local}" for key, local in p["names"].items()}
        self.w: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden
        kd = self.G * self.D
        small = dict(role="small32", tag="recurrent")
        rows = (("q", kd), ("k", kd), ("v", self.inner), ("decay_down", self.low), ("gate_down", self.gate_low),
                ("beta", self.heads))
        convs = (("q_conv", kd), ("k_conv", kd), ("v_conv", self.inner))
        return [
            TensorSpec(n["in"], (sum(r for _, r in rows), H),
                       sources=(Cat(tuple(Name(n[key], (r, H)) for key, r in rows), 0),)),
            TensorSpec(n["conv"], (self.conv_channels, self.taps), init=Init(0.0, 0.3),
                       sources=(Cat(tuple(Name(n[key], (r, self.taps)) for key, r in convs), 0),), **small),
            TensorSpec(n["decay_up"], (self.heads * self.D, self.low), init=Init(0.0, 0.2)),
            TensorSpec(n["gate_up"], (self.inner, self.gate_low), init=Init(0.0, 0.2)),
            TensorSpec(n["a_log"], (self.heads,), init=Init(-1.0, 0.5), **small),
            TensorSpec(n["dt_bias"], (self.heads * self.D,), init=Init(-1.0, 0.5), **small),
            TensorSpec(n["norm"], (self.P,), role="small32", init=Init(1.0, 0.0), tag="norm"),
            TensorSpec(n["o"], (H, self.inner), tag="residual_out"),
        ]

    def bind(self, tensors, dtype) -> None:
        self.w = {key: tensors[self.names[key]]
                  for key in ("in", "conv", "decay_up", "gate_up", "a_log", "dt_bias", "norm", "o")}

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T, ws, w = x.shape[0], ctx.workspace, self.w
        C, inner, heads, low = self.conv_channels, self.inner, self.heads, self.low
        both = low + self.gate_low
        conv_state, state = self._states(cache)
        proj = linear.linear(x, w["in"], ws.get("cdelta.in", (T, C + both + heads), ctx.dtype))
        qkv = ws.get("cdelta.qkv", (T, C), ctx.dtype)
        ops.conv_silu(proj[:, :C], qkv, w["conv"], None, conv_state, ctx.token_seg, ctx.seg_slot,
                      ctx.seg_q_start)
        # the decay's second step leaves its float32 accumulator: softplus and exp follow in float32
        decay = linear.linear(proj[:, C:C + low], w["decay_up"], ws.get("cdelta.decay", (T, heads * self.D),
                                                                        torch.float32))
        gate = linear.linear(proj[:, C + low:C + both], w["gate_up"], ws.get("cdelta.gate", (T, inner), ctx.dtype))
        o = ws.get("cdelta.o", (T, inner), torch.float32)
        ops.channel_delta_scan(qkv, proj[:, C + both:], decay, w["dt_bias"], w["a_log"], state, o, ctx.seg_slot,
                               ctx.seg_q_start, heads, self.G, self.D, self.P, self.unit_eps, self.D ** -0.5)
        gated = ws.get("cdelta.gated", (T, inner), ctx.dtype)
        ops.gated_norm(o, gate, w["norm"], gated, heads, self.eps, gate_first=False, gate_kind="sigmoid")
        if out is None:
            out = ws.get("cdelta.out", (T, self.hidden), ctx.dtype)
        return linear.linear(gated, w["o"], out)


@register_mixer("retention")
class Retention(_Recurrent):
    """params: ``hidden_size, heads, key_dim, head_dim, decay`` (one constant per head), ``norm_eps``,
    ``position`` (a PartSpec: which leading dimensions of a q / k head turn, in halves), ``scope`` and
    ``names`` (q, k, v, gate, o and the merged input projection ``in``).  k is multiplied by ``key_dim
    ** -0.5`` after the rotation; the read-out of a head is divided by its root mean square (no
    weight), the row gated by ``silu(W_g h)``."""

    taps = 1
    conv_channels = 0

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.D = int(p["key_dim"])
        self.P = int(p["head_dim"])
        self.eps = float(p["norm_eps"])
        self.decay_values = [float(v) for v in p["decay"]]
        if len(self.decay_values) != self.heads or self.D > 256:
            raise ValueError("retention: one decay per head, key_dim at most 256")
        pos_spec = p["position"]
        self.position = POSITIONS.get(pos_spec.kind)(pos_spec, prefix)
        if self.position.rotary_dim and self.position.interleaved:
            raise ValueError("retention: the scan turns dimension i with i + half only")
        self.inner = self.heads * self.P
        self.state_values = self.heads * self.D * self.P
        scope = self.name(p["scope"])
        self.names = {key: f"{scope}.{local}" for key, local in p["names"].items()}
        self.w: Dict[str, torch.Tensor] = {}
        self.decay = self.ones = None

    def children(self):
        return [self.position]

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden
        kd = self.heads * self.D
        rows = (("q", kd), ("k", kd), ("v", self.inner), ("gate", self.inner))
        return [
            TensorSpec(n["in"], (sum(r for _, r in rows), H),
                       sources=(Cat(tuple(Name(n[key], (r, H)) for key, r in rows), 0),)),
            TensorSpec(n["o"], (H, self.inner), tag="residual_out"),
        ]

    def bind(self, tensors, dtype) -> None:
        self.w = {key: tensors[self.names[key]] for key in ("in", "o")}
        device = self.w["in"].device
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)
        self.ones = torch.ones(self.P, dtype=torch.float32, device=device)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T, ws, w = x.shape[0], ctx.workspace, self.w
        inner, kd = self.inner, self.heads * self.D
        _, state = self._states(cache)
        proj = linear.linear(x, w["in"], ws.get("retention.in", (T, 2 * kd + 2 * inner), ctx.dtype))
        o = ws.get("retention.o", (T, inner), torch.float32)
        ops.retention_scan(proj[:, :2 * kd + inner], self.decay, self.position.table(ctx.device, ctx.max_positions),
                           ctx.seg_pos0, state, o, ctx.seg_slot, ctx.seg_q_start, self.heads, self.D, self.P,
                           self.D ** -0.5)
        gated = ws.get("retention.gated", (T, inner), ctx.dtype)
        ops.gated_norm(o, proj[:, 2 * kd + inner:], self.ones, gated, self.heads, self.eps, gate_first=False)
        if out is None:
            out = ws.get("retention.out", (T, self.hidden), ctx.dtype)
        return linear.linear(gated, w["o"], out)
