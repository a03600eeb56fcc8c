"""Attention mixers that keep ONE tensor per token in the cache.

Both run causal softmax attention through the kernels of :mod:`.attention`
over pages that hold a single plane, read as keys and again as values.

``shared_kv_attention`` - grouped-query attention whose values are its keys::

    q_t = Wq h_t  (heads x dim),   k_t = Wk h_t  (kv_heads x dim),   v_t = k_t
    q_t <- q_t * (1 + coef * ln(floor((t + 1) / every) + 1))      (query temperature)
    o_t,i = sum_{j <= t} softmax_j(q_t,i . k_j,g(i) * scale) k_j,g(i);   y_t = Wo o_t

No rotation: the temperature is the only way a position enters.

``latent_attention`` - keys and values are made from a cached latent vector::

    c_t = rms(Wdkv h_t) * w_c                (rank numbers: all the cache keeps)
    k_j,i = Wuk,i c_j,   v_j,i = Wuv,i c_j,   score = q_t,i . k_j,i * scale
    o_t,i = sigmoid(Wg h_t)_i * sum_j softmax_j(score) v_j,i;   y_t = Wo o_t

Since ``q . (Wuk c) = (Wuk^T q) . c`` and ``sum_j p_j Wuv c_j = Wuv (sum_j p_j c_j)``,
the mixer multiplies the queries by ``Wuk^T`` per head, attends over the latent
pages as ONE shared key/value head of size ``rank``, and multiplies the result by
``Wuv`` per head: the keys and values themselves are never formed, for a prompt
portion no more than for a decoded token, so the logits at a position do not
depend on how the prompt was cut.

``latent_attention`` also takes the fuller form of the same idea: queries through a normed latent
of their own (``c_q = rms(Wdq h) w_q``, ``q = Wuq c_q``), a key part of ``rot_dim`` values that is not
made from the latent but projected directly, rotated by the position and shared by all heads (every
head's query carries ``rot_dim`` rotated values for it), a sliding window, and a gate per output
value instead of per head::

    score = (q_i[:dq] . Wuk,i c_j + rot(q_i[dq:]) . rot(k_j)) * scale

The cache keeps ``[c_j | rot(k_j)]`` per token, the absorbed query is ``[Wuk,i^T q_i[:dq] | rot(q_i[dq:])]``,
and attention runs over rows of ``rank + rot_dim`` values, of which the first ``rank`` are the "values".

The reference's models have neither mixer; its attention layer
(python/freetoken/models/minimax_m2/attention.py:29-84) is the pattern both follow.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..cache.manager import PagedKeyNeed
from ..csrc import ops
from ..weights.spec import Cat, Init, Name, TensorSpec
from . import linear
from .attention import PagedSoftmaxCore
from .base import POSITIONS, CacheView, Mixer, StepContext, register_mixer


def _both_planes(pages: torch.Tensor) -> torch.Tensor:
    """``[pages, kv_heads, page, d]`` seen as the kernels' ``[2 (K, V), ...]``: the same
    plane twice."""
    return pages.unsqueeze(0).expand(2, *pages.shape)


@register_mixer("shared_kv_attention")
class SharedKVAttention(PagedSoftmaxCore, Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, head_dim, sm_scale``,
    ``q_temp_coef`` (0: no temperature), ``q_temp_every``, ``sliding_window`` (None: all
    keys), ``scope`` and ``names`` (q, k, o and the merged qk tensor below the scope)."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.scale = float(p["sm_scale"])
        self.temp_coef = float(p.get("q_temp_coef", 0.0))
        self.temp_every = int(p.get("q_temp_every", 1))
        self.window = p.get("sliding_window")
        if self.nkv <= 0 or self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} is not a multiple of num_kv_heads {self.nkv}")
        if self.d > 1024:
            raise ValueError(f"head_dim {self.d} exceeds what the attention kernels take (1024)")
        if self.temp_coef != 0.0 and self.temp_every <= 0:
            raise ValueError("q_temp_every must be positive")
        names = p["names"]
        scope = self.name(p["scope"])
        self.n_qk = f"{scope}.{names['qk']}"
        self.n_q, self.n_k, self.n_o = (f"{scope}.{names[k]}" for k in ("q", "k", "o"))
        self.w_qk = self.w_o = None

    def cache_need(self):
        return PagedKeyNeed(self.nkv, self.d, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        qn, kn = self.nq * self.d, self.nkv * self.d
        return [
            TensorSpec(self.n_qk, (qn + kn, self.hidden), sources=(Cat((
                Name(self.n_q, (qn, self.hidden)), Name(self.n_k, (kn, self.hidden))), 0),)),
            TensorSpec(self.n_o, (self.hidden, qn), tag="residual_out"),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.w_qk = tensors[self.n_qk]
        self.w_o = tensors[self.n_o]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] + self.attention_libraries(dtype) + linear.libraries(dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        qn, kn = self.nq * self.d, self.nkv * self.d
        qk = linear.linear(x, self.w_qk, ws.get("kattn.qk", (T, qn + kn), ctx.dtype))
        q = ws.get("kattn.q", (T, qn), ctx.dtype)
        table = ctx.block_tables[cache.block_table_index]
        ops.key_store(qk, q, cache.pages if cache.writes else None, None, ctx.token_pos, ctx.token_seg,
                      table, q_off=0, k_off=qn, num_heads=self.nq, q_dim=self.d, num_kv_heads=self.nkv,
                      k_dim=self.d, temp_coef=self.temp_coef, temp_every=self.temp_every)
        o = ws.get("kattn.o", (T, qn), ctx.dtype)
        self.attend(ctx, q, o, _both_planes(cache.pages), table)
        if out is None:
            out = ws.get("kattn.y", (T, self.hidden), ctx.dtype)
        return linear.linear(o, self.w_o, out)


@register_mixer("latent_attention")
class LatentAttention(PagedSoftmaxCore, Mixer):
    """params: ``hidden_size, num_heads, qk_dim, v_dim, rank, sm_scale, norm_eps``,
    ``output_gate`` (a sigmoid gate per head, read from the mixer's input),
    ``scope`` and ``names`` (q, down, gate, latent_norm, up_k, up_v, o and the merged input
    projection below the scope).

    Options of the fuller form (module docstring): ``q_rank`` (queries through a normed latent of
    that size; ``names`` then also has q_down, q_norm, q_up), ``rot_dim`` with ``position`` (a PartSpec;
    the rotated key part and the rotated tail of every head's query), ``sliding_window``, ``gate_per``
    (``"head"``, the default, or ``"element"``: one gate per output value)."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = 1                       # every head attends over the one latent
        self.dq = int(p["qk_dim"])
        self.dv = int(p["v_dim"])
        self.d = self.rank = int(p["rank"])
        self.scale = float(p["sm_scale"])
        self.eps = float(p["norm_eps"])
        self.gated = bool(p.get("output_gate", True))
        self.window = p.get("sliding_window")
        self.q_rank = int(p["q_rank"]) if p.get("q_rank") else None
        self.rot = int(p.get("rot_dim") or 0)
        self.gate_per = str(p.get("gate_per", "head"))
        if self.gate_per not in ("head", "element"):
            raise ValueError("gate_per must be 'head' or 'element'")
        self.d = self.rank + self.rot          # a cached row, and the head size the kernels see
        self.position = None
        if self.rot:
            pos_spec = p["position"]
            self.position = POSITIONS.get(pos_spec.kind)(pos_spec, prefix)
            if self.position.rotary_dim != self.rot:
                raise ValueError(f"latent_attention: the position part turns {self.position.rotary_dim} "
                                 f"dimensions, the rotated key part has {self.rot}")
        self.full = bool(self.rot or self.q_rank or self.gate_per == "element")
        if self.d > 1024:
            raise ValueError(f"latent rank plus rotated part {self.d} exceeds what the attention kernels take (1024)")
        names = p["names"]
        scope = self.name(p["scope"])
        self.n = {k: f"{scope}.{v}" for k, v in names.items()}
        self.w_in = self.w_norm = self.w_uk = self.w_uv = self.w_ukt = self.w_o = None
        self.w_qnorm = self.w_uq = None

    def children(self):
        return [self.position] if self.position is not None else []

    def cache_need(self):
        return PagedKeyNeed(1, self.d, self.window)

    def _gate_width(self) -> int:
        if not self.gated:
            return 0
        return self.nq if self.gate_per == "head" else self.nq * self.dv

    def tensor_specs(self) -> List[TensorSpec]:
        H, W, R = self.nq, self.hidden, self.rank
        q_width = H * (self.dq + self.rot)
        if self.q_rank:
            pieces = [Name(self.n["q_down"], (self.q_rank, W))]
        else:
            pieces = [Name(self.n["q"], (q_width, W))]
        pieces.append(Name(self.n["down"], (R + self.rot, W)))
        if self.gated:
            pieces.append(Name(self.n["gate"], (self._gate_width(), W)))
        specs = [
            TensorSpec(self.n["in"], (sum(piece.shape[0] for piece in pieces), W), sources=(Cat(tuple(pieces), 0),)),
            TensorSpec(self.n["latent_norm"], (R,), role="small32", init=Init(mean=1.0, std=0.0), tag="norm"),
            TensorSpec(self.n["up_k"], (H * self.dq, R)),
            TensorSpec(self.n["up_v"], (H * self.dv, R)),
            TensorSpec(self.n["o"], (W, H * self.dv), tag="residual_out"),
        ]
        if self.q_rank:
            specs += [TensorSpec(self.n["q_norm"], (self.q_rank,), role="small32", init=Init(mean=1.0, std=0.0),
                                 tag="norm"),
                      TensorSpec(self.n["q_up"], (q_width, self.q_rank))]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        H, R = self.nq, self.rank
        self.w_in = tensors[self.n["in"]]
        self.w_norm = tensors[self.n["latent_norm"]]
        self.w_uk = tensors[self.n["up_k"]].view(H, self.dq, R)      # [head][dq, R]
        self.w_uv = tensors[self.n["up_v"]].view(H, self.dv, R)      # [head][dv, R]
        # the CUDA-core product wants [N, K] rows: Wuk^T per head
        self.w_ukt = self.w_uk.transpose(1, 2).contiguous() if dtype == torch.float32 else None
        self.w_o = tensors[self.n["o"]]
        if self.q_rank:
            self.w_qnorm = tensors[self.n["q_norm"]]
            self.w_uq = tensors[self.n["q_up"]]

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"] + self.attention_libraries(dtype) + linear.libraries(dtype)

    def _forward_full(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        """The fuller form: a query latent, a rotated key part, a window, a gate per value."""
        T, ws = x.shape[0], ctx.workspace
        H, R, dq, dv, rot, d = self.nq, self.rank, self.dq, self.dv, self.rot, self.d
        z = linear.linear(x, self.w_in, ws.get("lattn.in", (T, self.w_in.shape[0]), ctx.dtype))
        q_width = H * (dq + rot)
        if self.q_rank:
            cq = ws.get("lattn.cq", (T, self.q_rank), ctx.dtype)
            ops.rms_rows(z[:, :self.q_rank], self.w_qnorm, cq, self.eps)
            q = linear.linear(cq, self.w_uq, ws.get("lattn.q_up", (T, q_width), ctx.dtype))
            at = self.q_rank
        else:
            q, at = z[:, :q_width], q_width
        table = ctx.block_tables[cache.block_table_index]
        q_abs = ws.get("lattn.q", (T, H, d), ctx.dtype)
        cos_sin = self.position.table(ctx.device, ctx.max_positions) if rot else None
        ops.latent_store(z[:, at:at + R + rot], q, q_abs, cache.pages if cache.writes else None, self.w_norm,
                         cos_sin, ctx.token_pos, ctx.token_seg, table, heads=H, q_dim=dq, rank=R, rot=rot,
                         interleaved=bool(rot and self.position.interleaved), eps=self.eps)
        # the unrotated part of every head's query into the latent's space: Wuk^T q per head
        q_heads = q.view(T, H, dq + rot)[:, :, :dq] if q.is_contiguous() else \
            q.unflatten(1, (H, dq + rot))[:, :, :dq]
        if ctx.dtype == torch.float32:
            ops.gemm_heads(q_heads, self.w_ukt, q_abs[:, :, :R])
        else:
            torch.bmm(q_heads.transpose(0, 1), self.w_uk, out=q_abs[:, :, :R].transpose(0, 1))
        o = ws.get("lattn.o", (T, H * d), ctx.dtype)
        self.attend(ctx, q_abs.view(T, H * d), o, _both_planes(cache.pages), table)
        # the first rank values of a head's result are the weighted latents: Wuv per head, then the gate
        y = ws.get("lattn.v", (T, H * dv), ctx.dtype)
        o_latent = o.view(T, H, d)[:, :, :R]
        if ctx.dtype == torch.float32:
            ops.gemm_heads(o_latent, self.w_uv, y.view(T, H, dv))
        else:
            torch.bmm(o_latent.transpose(0, 1), self.w_uv.transpose(1, 2), out=y.view(T, H, dv).transpose(0, 1))
        if self.gated:
            gate = z[:, at + R + rot:]
            if self.gate_per == "head":
                ops.gate_heads(y, gate, H, dv)
            else:
                ops.gate_heads(y, gate, H * dv, 1)
        if out is None:
            out = ws.get("lattn.y", (T, self.hidden), ctx.dtype)
        return linear.linear(y, self.w_o, out)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        if self.full:
            return self._forward_full(ctx, x, cache, out)
        T = x.shape[0]
        ws = ctx.workspace
        H, R, dq, dv = self.nq, self.rank, self.dq, self.dv
        width = self.w_in.shape[0]
        z = linear.linear(x, self.w_in, ws.get("lattn.in", (T, width), ctx.dtype))
        table = ctx.block_tables[cache.block_table_index]
        # the latent: RMS norm in float32, into the token's place of the page
        ops.key_store(z, None, cache.pages if cache.writes else None, self.w_norm, ctx.token_pos,
                      ctx.token_seg, table, q_off=0, k_off=H * dq, num_heads=H, q_dim=dq, num_kv_heads=1,
                      k_dim=R, eps=self.eps)
        # queries into the latent's space: q' = Wuk^T q per head
        q = ws.get("lattn.q", (T, H * R), ctx.dtype)
        q_heads = z[:, :H * dq].view(T, H, dq)
        if ctx.dtype == torch.float32:
            ops.gemm_heads(q_heads, self.w_ukt, q.view(T, H, R))
        else:
            torch.bmm(q_heads.transpose(0, 1), self.w_uk, out=q.view(T, H, R).transpose(0, 1))
        o = ws.get("lattn.o", (T, H * R), ctx.dtype)
        self.attend(ctx, q, o, _both_planes(cache.pages), table)
        # back out of the latent's space: Wuv per head, then the gate
        y = ws.get("lattn.v", (T, H * dv), ctx.dtype)
        if ctx.dtype == torch.float32:
            ops.gemm_heads(o.view(T, H, R), self.w_uv, y.view(T, H, dv))
        else:
            torch.bmm(o.view(T, H, R).transpose(0, 1), self.w_uv.transpose(1, 2),
                      out=y.view(T, H, dv).transpose(0, 1))
        if self.gated:
            ops.gate_heads(y, z[:, H * dq + R:], H, dv)
        if out is None:
            out = ws.get("lattn.y", (T, self.hidden), ctx.dtype)
        return linear.linear(y, self.w_o, out)
