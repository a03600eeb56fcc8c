"""Grouped-query softmax attention over the paged cache.

Per token: ``qkv = x @ Wqkv^T`` (one merged product, no bias), optional QK
RMSNorm (over the whole q / k projection, or per head), rotary on the first
``rotary_dim`` dims of each head, K and V stored into the request's pages,
causal softmax attention with scale ``sm_scale`` over the cached keys (all of
them, or the latest ``sliding_window``), then ``@ Wo^T``.

Options no model of the reference has, each a parameter of the mixer: a short causal
convolution per channel behind the q, k and v projections (its last inputs per request in a
state slot); a mask in chunks (a query sees the keys of its own chunk of positions); scores
capped by ``cap * tanh(s / cap)``; a sink in the softmax's denominator, a fixed score or a
learned one per head; a sigmoid gate on the heads' outputs, one per head or one per value, read
from the mixer's input by the same merged product.

Reference: python/freetoken/models/minimax_m2/attention.py:29-84 (merged QKV,
per-layer norm, rotary, backend call, o_proj),
python/freetoken/models/minimax_m3/attention.py:54-56,90-92 (per-head norm),
python/freetoken/attention/triton.py:150-216 (store, then decode / extend
kernels), python/freetoken/kernel/triton/attention.py:74,118-139 (mask, scale,
softmax).
"""

from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from ..cache.manager import CompositeNeed, PagedKVNeed, StateNeed
from ..csrc import ops
from ..weights.spec import Cat, Init, Name, TensorSpec
from . import linear
from .base import POSITIONS, CacheView, Mixer, StepContext, StepPlan, StepShape, register_mixer

# query tokens per tile of the prefill attention kernels' tile list
PREFILL_TILE = 64

_NORM_MODES = {"none": 0, "per_layer": 1, "per_head": 2}


class PagedSoftmaxCore:
    """What every mixer shares that runs causal softmax attention over paged keys and
    values: the step metadata of the attention kernels and the choice among them.  A
    mixer that mixes this in states ``nq`` (query heads), ``nkv`` (KV heads), ``d`` (head
    size as the kernels see it), ``scale`` and ``window``."""

    nq: int
    nkv: int
    d: int
    scale: float
    window = None
    # what else happens to the scores (chunks, cap, sink): ops.ScoreOptions, None: nothing
    options = None

    # ---- step metadata ---------------------------------------------------------
    def step_plan_key(self):
        # the lists depend on the step's segments only: every attention layer shares them
        return "paged_attention"

    def plan_step(self, shape: StepShape) -> StepPlan:
        """What the attention kernels want to know about a step: which token rows
        are single-token segments (decode kernel; listed only when the step also
        has longer segments, otherwise it is all rows), the 64-token query tiles
        of the longer segments (prefill kernels: segment and first token inside
        it), how many query-key pairs those score, and the longest context of a
        decode row (in whole block-table rows for a decode-only step, so that the
        split count - and with it a captured graph - stays put while contexts grow)."""
        segs = shape.segments
        dec = [s.q_start for s in segs if s.n == 1]
        tiles = [(i, q0) for i, s in enumerate(segs) if s.n > 1 for q0 in range(0, s.n, PREFILL_TILE)]
        arrays = {
            "tile_seg": np.asarray([t[0] for t in tiles], dtype=np.int32),
            "tile_q0": np.asarray([t[1] for t in tiles], dtype=np.int32),
        }
        if dec and tiles:
            arrays["decode_rows"] = np.asarray(dec, dtype=np.int32)
        if shape.max_q_len == 1:
            max_decode_kv = shape.table_width * shape.page_size
        else:
            max_decode_kv = max((s.pos0 + 1 for s in segs if s.n == 1), default=0)
        host = {
            "num_decode_rows": len(dec),
            "num_prefill_tiles": len(tiles),
            "prefill_scores": sum(s.n * (s.pos0 + (s.n + 1) // 2) for s in segs if s.n > 1),
            "max_decode_kv_len": max_decode_kv,
        }
        return StepPlan(arrays=arrays, host=host)

    def attention_libraries(self, dtype, d: int = 0) -> List[str]:
        d = d or self.d
        fast = []
        if dtype == torch.bfloat16 and d in ops.DECODE_HEAD_DIMS:
            fast = ["attention_decode", "attention_prefill"]
        if fast and d in (64, 128):
            # TMA-fed kernels (the prefill one also builds the tensor maps both use)
            fast += ["attention_prefill_tc", "attention_decode_tma"]
        return ["attention_simt"] + fast

    def attend(self, ctx: StepContext, q, o, kv_pages, table) -> None:
        """Single-token rows go to the split-KV tensor-core kernel, rows of
        longer segments to a prefill kernel; sizes those refuse (and the
        float32 path) go to the generic kernel.  ``kv_pages`` is ``[2 (K, V),
        pages, kv_heads, page, head_dim]``."""
        if ops.attn_decode_takes(q, self.d):
            plan = ctx.plan(self)
            n_dec, n_tiles = plan.host["num_decode_rows"], plan.host["num_prefill_tiles"]
            if n_dec > 0:
                ops.attn_decode(q, o, kv_pages, plan.tensors.get("decode_rows"), n_dec,
                                ctx.token_pos, ctx.token_seg, table, self.nq, self.nkv, self.d,
                                self.scale, self.window, plan.host["max_decode_kv_len"], ctx.workspace,
                                options=self.options)
            if n_tiles > 0:
                tile_seg, tile_q0 = plan.tensors["tile_seg"], plan.tensors["tile_q0"]
                if (plan.host["prefill_scores"] >= ops.PREFILL_TC_MIN_SCORES
                        and ops.attn_prefill_tc_takes(q, kv_pages, self.d, self.window)):
                    ops.attn_prefill_tc(q, o, kv_pages, tile_seg, tile_q0, ctx.seg_q_start,
                                        ctx.seg_pos0, table, self.nq, self.nkv, self.d, self.scale, self.window,
                                        options=self.options)
                    return
                ops.attn_prefill(q, o, kv_pages, tile_seg, tile_q0, ctx.seg_q_start, ctx.seg_pos0,
                                 table, self.nq, self.nkv, self.d, self.scale, self.window, options=self.options)
            return
        ops.attn_paged_simt(q, o, kv_pages, ctx.token_pos, ctx.token_seg, table,
                            self.nq, self.nkv, self.d, self.scale, self.window, options=self.options)


@register_mixer("paged_attention")
class PagedAttention(PagedSoftmaxCore, Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, head_dim, sm_scale,
    qk_norm`` (none | per_layer | per_head), ``qk_norm_eps, qk_norm_plus_one,
    sliding_window`` (None: all keys), ``position`` (a PartSpec), ``scope`` and
    ``checkpoint_names`` (q, k, v, o, fused qkv, q_norm, k_norm tensor names
    below the scope).

    ``value_dim`` (default ``head_dim``): the size of a value head where it differs from the
    size of a query / key head.  The kernels see heads of the larger size: the smaller
    projection's matrix (and the output projection's columns) are filled up with zeros when
    the weights are bound, which changes no score and no output and costs cache and
    arithmetic only where the two sizes differ.  ``bias`` (default False): the q, k, v and o
    projections add a bias (``checkpoint_names`` then also has q_bias, k_bias, v_bias, o_bias
    and the fused qkv_bias).

    ``conv_taps`` (default 0): q, k and v each pass a causal convolution over time per channel
    (``checkpoint_names`` q_conv, k_conv, v_conv: ``[channels, taps]``, the last column weighing
    the current token; no bias, no activation) directly behind the projection; the last
    ``conv_taps - 1`` projected rows of a request live in a state slot.  ``chunk``: a query sees
    only keys of its own chunk of that many positions.  ``softcap``: scores become ``cap *
    tanh(score / cap)``.  ``sink_value`` (a fixed score) or ``sink`` (True: a learned score per
    head, ``checkpoint_names`` sink): a score without key or value in the softmax's denominator.
    ``gate`` (``"head"`` or ``"element"``): the heads' outputs times ``sigmoid(Wg x)``, one gate
    per head or per value (``checkpoint_names`` gate), merged into the qkv product.
    ``fill_heads`` (default False): in bfloat16, heads of up to 128 values that are no size of the
    tensor-core attention kernels (32, 64, 128) are filled up with zeros to the next one, exactly as
    heads are filled up to the larger of key and value size: a model with heads of 112 values then
    runs its prompts and decoded tokens on the tensor-core kernels with heads of 128, at the price
    of a seventh more cache and arithmetic in the mixer.  float32 keeps the sizes as they are."""

    graph_capturable = True
    writes_into_out = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.dk = int(p["head_dim"])
        self.dv = int(p.get("value_dim") or self.dk)
        self.d = max(self.dk, self.dv)          # the head size the kernels and the cache see (bind may fill it up)
        self.fill_heads = bool(p.get("fill_heads", False))
        self.has_bias = bool(p.get("bias", False))
        self.scale = float(p["sm_scale"])
        self.norm_mode = _NORM_MODES[p.get("qk_norm", "none")]
        self.norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.norm_plus_one = bool(p.get("qk_norm_plus_one", False))
        self.window = p.get("sliding_window")
        self.chunk = int(p.get("chunk") or 0)
        self.softcap = float(p.get("softcap") or 0.0)
        self.sink_value = p.get("sink_value")
        self.learned_sink = bool(p.get("sink", False))
        self.gate = p.get("gate")
        self.taps = int(p.get("conv_taps") or 0)
        if self.gate not in (None, "head", "element"):
            raise ValueError("gate must be None, 'head' or 'element'")
        if self.window and self.chunk:
            raise ValueError("a sliding window and a mask in chunks exclude each other")
        if self.learned_sink and self.sink_value is not None:
            raise ValueError("a sink is a fixed score or a learned one per head, not both")
        if self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} is not a multiple of num_kv_heads {self.nkv}")
        if self.d > 1024:
            raise ValueError(f"head size {self.d} exceeds what the attention kernels take (1024)")
        if self.dk != self.dv and self.norm_plus_one and self.dk < self.d:
            raise ValueError("a one-plus QK norm over heads that are filled up to the value size is not offered")
        pos_spec = p["position"]
        self.position = POSITIONS.get(pos_spec.kind)(pos_spec, prefix)
        scope = p["scope"]
        names = p["checkpoint_names"]
        self.scope = self.name(scope)
        self.n_qkv = f"{self.scope}.{names['qkv']}"
        self.n_o = f"{self.scope}.{names['o']}"
        self.n_qnorm = f"{self.scope}.{names['q_norm']}"
        self.n_knorm = f"{self.scope}.{names['k_norm']}"
        self._split = [f"{self.scope}.{names[k]}" for k in ("q", "k", "v")]
        self.w_qkv = self.w_o = self.w_qnorm = self.w_knorm = self.b_qkv = self.b_o = None
        self.n_gate = f"{self.scope}.{names['gate']}" if self.gate else None
        self.n_sink = f"{self.scope}.{names['sink']}" if self.learned_sink else None
        self.n_conv = f"{self.scope}.{names.get('qkv_conv', 'qkv.conv')}" if self.taps else None
        self._split_conv = [f"{self.scope}.{names[k]}" for k in ("q_conv", "k_conv", "v_conv")] if self.taps else []
        self.w_conv = self.w_sink = None
        self.gate_width = 0 if not self.gate else (self.nq if self.gate == "head" else self.nq * self.dv)
        if self.gate and self.has_bias:
            raise ValueError("a gate merged into a biased qkv product is not offered")
        if self.has_bias:
            self.n_qkv_bias = f"{self.scope}.{names['qkv_bias']}"
            self.n_o_bias = f"{self.scope}.{names['o_bias']}"
            self._split_bias = [f"{self.scope}.{names[k]}" for k in ("q_bias", "k_bias", "v_bias")]

    def children(self):
        return [self.position]

    # ---- cache and weights ------------------------------------------------
    def cache_need(self):
        # keys of chunks that are over are never read again: the pages behind the last `chunk`
        # positions go back to the pool like those behind a window
        paged = PagedKVNeed(self.nkv, self.d, self.window or (self.chunk or None))
        if self.taps > 1:
            return CompositeNeed((paged, StateNeed(((self.taps - 1) * (self.nq + 2 * self.nkv) * self.d,))))
        return paged

    def tensor_specs(self) -> List[TensorSpec]:
        qn, kn, vn = self.nq * self.dk, self.nkv * self.dk, self.nkv * self.dv
        pieces = [Name(self._split[0], (qn, self.hidden)), Name(self._split[1], (kn, self.hidden)),
                  Name(self._split[2], (vn, self.hidden))]
        if self.gate:
            pieces.append(Name(self.n_gate, (self.gate_width, self.hidden)))
        specs = [
            TensorSpec(self.n_qkv, (qn + kn + vn + self.gate_width, self.hidden), sources=(Cat(tuple(pieces), 0),)),
            TensorSpec(self.n_o, (self.hidden, self.nq * self.dv), tag="residual_out"),
        ]
        if self.taps:
            specs.append(TensorSpec(self.n_conv, (qn + kn + vn, self.taps), role="small32",
                                    init=Init(mean=0.0, std=self.taps ** -0.5), tag="conv", sources=(Cat((
                                        Name(self._split_conv[0], (qn, self.taps)),
                                        Name(self._split_conv[1], (kn, self.taps)),
                                        Name(self._split_conv[2], (vn, self.taps))), 0),)))
        if self.learned_sink:
            specs.append(TensorSpec(self.n_sink, (self.nq,), role="small32", init=Init(mean=0.0, std=1.0), tag="sink"))
        if self.has_bias:
            specs.append(TensorSpec(self.n_qkv_bias, (qn + kn + vn,), role="small32", tag="bias", sources=(Cat((
                Name(self._split_bias[0], (qn,)), Name(self._split_bias[1], (kn,)),
                Name(self._split_bias[2], (vn,))), 0),)))
            specs.append(TensorSpec(self.n_o_bias, (self.hidden,), role="small32", tag="bias"))
        if self.norm_mode:
            sizes = (qn, kn) if self.norm_mode == 1 else (self.dk, self.dk)
            mean = 0.0 if self.norm_plus_one else 1.0
            for name, size in zip((self.n_qnorm, self.n_knorm), sizes):
                specs.append(TensorSpec(name, (size,), role="small32",
                                        init=Init(mean=mean, std=0.0), tag="norm"))
        return specs

    def _filled(self, t: torch.Tensor, heads_and_sizes, axis: int) -> torch.Tensor:
        """``t`` with every head along ``axis`` filled up with zeros to the kernels' head size;
        ``heads_and_sizes``: (heads, size) of the runs of heads along the axis, in order."""
        if all(size == self.d for _, size in heads_and_sizes):
            return t
        pieces, at = [], 0
        for heads, size in heads_and_sizes:
            run = t.narrow(axis, at, heads * size)
            at += heads * size
            shape = list(run.shape)
            shape[axis:axis + 1] = [heads, size]
            run = run.reshape(shape)
            pad = list(run.shape)
            pad[axis + 1] = self.d - size
            pieces.append(torch.cat((run, run.new_zeros(pad)), axis + 1).flatten(axis, axis + 1))
        return torch.cat(pieces, axis).contiguous()

    def _head_size(self, dtype) -> int:
        """The head size the kernels and the cache see for compute dtype ``dtype``."""
        d = max(self.dk, self.dv)
        if self.fill_heads and dtype == torch.bfloat16 and d <= max(ops.DECODE_HEAD_DIMS):
            return min(size for size in ops.DECODE_HEAD_DIMS if size >= d)
        return d

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.d = self._head_size(dtype)
        runs = ((self.nq, self.dk), (self.nkv, self.dk), (self.nkv, self.dv))
        gate_runs = () if not self.gate else (((self.nq, 1),) if self.gate == "head" else ((self.nq, self.dv),))
        if self.gate == "head":
            # one row per head: not a head's worth of values, nothing to fill up
            w = tensors[self.n_qkv]
            self.w_qkv = torch.cat((self._filled(w[:w.shape[0] - self.nq], runs, 0), w[w.shape[0] - self.nq:]), 0).contiguous()
        else:
            self.w_qkv = self._filled(tensors[self.n_qkv], runs + gate_runs, 0)
        self.w_o = self._filled(tensors[self.n_o], ((self.nq, self.dv),), 1)
        if self.has_bias:
            self.b_qkv = self._filled(tensors[self.n_qkv_bias], runs, 0)
            self.b_o = tensors[self.n_o_bias]
        if self.norm_mode == 1:
            self.w_qnorm = self._filled(tensors[self.n_qnorm], ((self.nq, self.dk),), 0)
            self.w_knorm = self._filled(tensors[self.n_knorm], ((self.nkv, self.dk),), 0)
        elif self.norm_mode:
            self.w_qnorm = self._filled(tensors[self.n_qnorm], ((1, self.dk),), 0)
            self.w_knorm = self._filled(tensors[self.n_knorm], ((1, self.dk),), 0)
        if self.taps:
            self.w_conv = self._filled(tensors[self.n_conv], runs, 0)
        if self.learned_sink:
            self.w_sink = tensors[self.n_sink]
        if self.chunk or self.softcap or self.learned_sink or self.sink_value is not None:
            self.options = ops.ScoreOptions(self.chunk, self.softcap, self.sink_value, self.w_sink)

    def libraries(self, dtype) -> List[str]:
        return (["elementwise"] + self.attention_libraries(dtype, self._head_size(dtype)) + linear.libraries(dtype, self.has_bias)
                + (["recurrent"] if self.taps else []) + (["rowwise"] if self.gate else []))

    # ---- forward ----------------------------------------------------------------
    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView, out=None) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        qn, kn = self.nq * self.d, self.nkv * self.d
        gw = self.gate_width if self.gate == "head" else (qn if self.gate else 0)
        qkv = linear.linear(x, self.w_qkv, ws.get("attn.qkv", (T, qn + 2 * kn + gw), ctx.dtype), bias=self.b_qkv)
        gate = qkv[:, qn + 2 * kn:] if self.gate else None
        if self.gate:
            qkv = qkv[:, :qn + 2 * kn]
        if self.taps > 1:
            cache, conv = cache.members
            mixed = ws.get("attn.conv", (T, qn + 2 * kn), ctx.dtype)
            if not cache.writes:
                raise ValueError("a mixer with a convolution's state cannot read another stop's cache")
            ops.conv_silu(qkv, mixed, self.w_conv, None, conv.state, ctx.token_seg, ctx.seg_slot, ctx.seg_q_start,
                          activation=False)
            qkv = mixed
        elif self.taps == 1:
            # one tap: a factor per channel, nothing carried from step to step
            mixed = ws.get("attn.conv", (T, qn + 2 * kn), ctx.dtype)
            ops.conv_silu(qkv, mixed, self.w_conv, None, ws.get("attn.no_state", (1, 1), torch.float32), ctx.token_seg,
                          ctx.seg_slot, ctx.seg_q_start, activation=False)
            qkv = mixed
        q = ws.get("attn.q", (T, qn), ctx.dtype)
        table = ctx.block_tables[cache.block_table_index]
        cos_sin = self.position.table(ctx.device, ctx.max_positions)
        ops.qk_rope_store(
            qkv, q, cache.kv_pages if cache.writes else None, self.w_qnorm, self.w_knorm,
            cos_sin, ctx.token_pos, ctx.token_seg, table, self.nq, self.nkv, self.d,
            self.position.rotary_dim, self.norm_mode, self.norm_plus_one,
            self.position.interleaved, self.norm_eps, norm_dim=self.dk)
        o = ws.get("attn.o", (T, qn), ctx.dtype)
        self.attend(ctx, q, o, cache.kv_pages, table)
        if self.gate == "head":
            ops.gate_heads(o, gate, self.nq, self.d)
        elif self.gate:
            ops.gate_heads(o, gate, qn, 1)
        if out is None:
            out = ws.get("attn.y", (T, self.hidden), ctx.dtype)
        return linear.linear(o, self.w_o, out, bias=self.b_o)
