"""Token embedding and output head.

Embedding: ``residual[t,:] = W[ids[t],:]`` with no scale
(python/freetoken/layers/embedding.py:39-47, kernel/csrc/jit/index.cu:31-59).
Head: ``logits = x @ Wlm^T`` in float32 for the rows asked for; with tied
weights ``Wlm`` is the embedding table (layers/embedding.py:107-115).

Options the reference's models do not have: an RMS norm of the embedded rows
(``residual[t,:] = rms(W[ids[t],:]) * g``, gathered and normed in one kernel), a cap on the
logits (``cap * tanh(logits / cap)``), a factor on the embedded row, and a second table whose row
is picked by a hash of the token and the one before it (``residual[t,:] = W[ids[t],:] * scale +
B[(ids[t-1] * mul_prev + ids[t] * mul_cur) mod buckets, :]``, row ``buckets`` for a sequence's
first token).  The token before a portion's first one is per-request state: the embedding
states a cache need like a mixer does, one int32 per request slot.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from ..weights.spec import Init, TensorSpec
from . import linear
from .base import CacheView, Embedding, Head, StepContext, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size, hidden_size``, ``scope`` (the table is ``<scope>.weight``) or
    ``tensor`` (its whole name); ``norm_tensor`` and ``norm_eps``: the embedded rows are
    RMS-normed with that weight before they become the residual stream.  ``scale`` (default 1):
    a factor on the embedded row.  ``pair_tensor`` with ``buckets, mul_prev, mul_cur``: a second
    table of ``buckets + 1`` rows, added by the hash of (previous token, token)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight_name = self.name(spec.get("tensor") or f"{spec.params['scope']}.weight")
        self.norm_name = self.name(spec.get("norm_tensor")) if spec.get("norm_tensor") else None
        self.norm_eps = float(spec.get("norm_eps", 1e-6))
        self.scale = float(spec.get("scale") if spec.get("scale") is not None else 1.0)
        self.pair_name = self.name(spec.get("pair_tensor")) if spec.get("pair_tensor") else None
        self.buckets = int(spec.get("buckets") or 0)
        self.mul_prev, self.mul_cur = int(spec.get("mul_prev") or 0), int(spec.get("mul_cur") or 0)
        if self.pair_name and self.buckets < 1:
            raise ValueError("a hashed second table needs 'buckets' >= 1")
        if self.norm_name and (self.pair_name or self.scale != 1.0):
            raise ValueError("an embedding norm beside a scale or a second table is not offered")
        self.weight = self.norm_weight = self.pair_weight = None

    def cache_need(self) -> Optional[StateNeed]:
        """The request's last token, where the second table's row depends on it."""
        return StateNeed((1,), "int32") if self.pair_name else None

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.weight_name, (self.vocab, self.hidden), tag="embedding")]
        if self.norm_name:
            specs.append(TensorSpec(self.norm_name, (self.hidden,), role="small32",
                                    init=Init(mean=1.0, std=0.0), tag="norm"))
        if self.pair_name:
            specs.append(TensorSpec(self.pair_name, (self.buckets + 1, self.hidden), tag="embedding"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]
        if self.norm_name:
            self.norm_weight = tensors[self.norm_name]
        if self.pair_name:
            self.pair_weight = tensors[self.pair_name]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] if (self.norm_name or self.pair_name or self.scale != 1.0) else ["elementwise"]

    def forward(self, ctx: StepContext, residual: torch.Tensor, cache: Optional[CacheView] = None) -> None:
        if self.pair_name or self.scale != 1.0:
            if self.pair_name and (cache is None or cache.state is None):
                raise ValueError("the hashed second table needs the embedding's per-request state")
            ops.embed_pair(ctx.token_ids, ctx.token_pos, ctx.token_seg, ctx.seg_slot, ctx.seg_q_start, self.weight,
                           self.pair_weight, cache.state if self.pair_name else None, residual, self.scale,
                           self.buckets, self.mul_prev, self.mul_cur)
        elif self.norm_name:
            ops.embed_norm(ctx.token_ids, self.weight, self.norm_weight, residual, self.norm_eps)
        else:
            ops.embed_gather(ctx.token_ids, self.weight, residual)


@register_head("lm_head")
class LMHead(Head):
    """params: ``vocab_size, hidden_size, scope`` (the tensor is ``<scope>.weight``) or ``tensor``
    (its whole name), ``tied_to`` (full name of
    the embedding table, or None; a tied head with no ``scope`` has no tensor of its own,
    not even an optional one), ``softcap`` (None or 0: no cap on the logits)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied_to = spec.get("tied_to")
        scope = spec.get("scope")
        own = spec.get("tensor") or (f"{scope}.weight" if scope else None)
        if not own and not self.tied_to:
            raise ValueError("a head needs a tensor of its own ('scope' or 'tensor') or a table to share "
                             "('tied_to')")
        self.own_name = self.name(own) if own else None
        self.weight_name = self.tied_to or self.own_name
        self.softcap = float(spec.get("softcap") or 0.0)
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.tied_to and not self.own_name:
            return []
        if self.tied_to:
            # a checkpoint of a tied model may still carry the head's tensor; it
            # is accepted and dropped (python/freetoken/layers/embedding.py:74-90)
            return [TensorSpec(self.own_name, (self.vocab, self.hidden), optional=True, keep=False)]
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]

    def libraries(self, dtype) -> List[str]:
        return linear.libraries(dtype) + (["rowwise"] if self.softcap else [])

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor) -> None:
        linear.linear(x, self.weight, out)
        if self.softcap:
            ops.softcap(out, self.softcap)
