"""A plain feed-forward: ``y = Wdown f(Wup h)``, or gated ``y = Wdown (f(Wgate h) * (Wup h))``.

``f`` is one of ``relu2`` (the square of relu), ``gelu_tanh`` and ``silu``,
evaluated in float32 on the up projection's output.  The reference's models
use gated, routed experts only (python/freetoken/layers/moe.py:83-92); its dense
linear layers (python/freetoken/layers/linear.py:31-32) are what this part is
made of.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from ..weights.spec import Cat, Name, TensorSpec
from . import linear
from .base import FeedForward, StepContext, register_feed_forward


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """params: ``hidden_size, intermediate_size, activation``, ``scope`` and ``names``
    (up, down below the scope); ``gated`` (default False): a gate projection beside the up
    projection (``names`` then also has gate, and gate_up for the merged matrix the model keeps).
    A gated feed-forward may also take the clamped pair ``swigluoai`` with ``act_alpha`` and
    ``act_limit``: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``, ``g sigmoid(alpha g) (u + 1)``."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.act = str(p.get("activation", "relu2"))
        self.act_alpha = float(p.get("act_alpha", 1.702))
        self.act_limit = float(p.get("act_limit", 7.0))
        known = ops.GLU_KINDS if p.get("gated", False) else ops.ACTIVATIONS
        if self.act not in known:
            raise ValueError(f"activation {self.act!r} is not one of {sorted(known)}")
        scope = self.name(p["scope"])
        self.n_up = f"{scope}.{p['names']['up']}"
        self.n_down = f"{scope}.{p['names']['down']}"
        self.gated = bool(p.get("gated", False))
        if self.gated:
            self.n_gate = f"{scope}.{p['names']['gate']}"
            self.n_gate_up = f"{scope}.{p['names']['gate_up']}"
        self.w_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        down = TensorSpec(self.n_down, (self.hidden, self.inter), tag="residual_out")
        if self.gated:
            shape = (self.inter, self.hidden)
            return [TensorSpec(self.n_gate_up, (2 * self.inter, self.hidden),
                               sources=(Cat((Name(self.n_gate, shape), Name(self.n_up, shape)), 0),)), down]
        return [TensorSpec(self.n_up, (self.inter, self.hidden)), down]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.w_up = tensors[self.n_gate_up if self.gated else self.n_up]
        self.w_down = tensors[self.n_down]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] + linear.libraries(dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor, out=None) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        if self.gated:
            # one product against [gate; up], then f(gate) * up in float32
            both = linear.linear(x, self.w_up, ws.get("mlp.gate_up", (T, 2 * self.inter), ctx.dtype))
            mid = ws.get("mlp.mid", (T, self.inter), ctx.dtype)
            ops.glu_rows(both, mid, self.act, self.act_alpha, self.act_limit)
            if out is None:
                out = ws.get("mlp.y", (T, self.hidden), ctx.dtype)
            return linear.linear(mid, self.w_down, out)
        # decode rows: the activation is the weight-streaming kernel's epilogue
        mid = linear.linear(x, self.w_up, ws.get("mlp.mid", (T, self.inter), ctx.dtype), activation=self.act)
        if out is None:
            out = ws.get("mlp.y", (T, self.hidden), ctx.dtype)
        return linear.linear(mid, self.w_down, out)
