"""RMSNorm with the residual add folded in.

``z = delta + residual; residual <- z; y = z * rsqrt(mean(z^2) + eps) * w``
in float32 (python/freetoken/kernel/triton/norm.py:101-112); ``plus_one``
selects the ``(1 + w)`` form (norm.py:69-72, python/freetoken/layers/norm.py:120-147).
The residual stream itself stays float32 between layers here (the reference
rounds it to the activation dtype each time it is stored, norm.py:108-109).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from ..weights.spec import Init, TensorSpec
from .base import Norm, StepContext, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``plus_one``, and ``scope`` (the tensor is ``<scope>.weight``
    below the prefix) or ``tensor`` (its whole name below the prefix)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.plus_one = bool(spec.get("plus_one", False))
        self.weight_name = self.name(spec.get("tensor") or f"{spec.params['scope']}.weight")
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        mean = 0.0 if self.plus_one else 1.0
        return [TensorSpec(self.weight_name, (self.size,), role="small32",
                           init=Init(mean=mean, std=0.0), tag="norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]

    def libraries(self, dtype) -> List[str]:
        return ["elementwise", "rowwise"]

    def forward(self, ctx: StepContext, delta, residual: torch.Tensor) -> torch.Tensor:
        out = ctx.workspace.get("norm.out", residual.shape, ctx.dtype)
        ops.rmsnorm(delta, residual, self.weight, out, self.eps, self.plus_one)
        return out

    def add_normed(self, ctx: StepContext, branch: torch.Tensor, residual: torch.Tensor, mult: float,
                   then: Optional["RMSNorm"] = None) -> Optional[torch.Tensor]:
        """``residual += mult * norm(branch)`` in float32, this norm being the branch's own
        (``branch`` is ``[T, H]`` or ``[T, k, H]`` partial rows, summed first).  With ``then`` the
        new residual rows are normed by that norm in the same launch and returned."""
        if then is None:
            ops.norm_add(branch, residual, self.weight, self.eps, self.plus_one, mult)
            return None
        out = ctx.workspace.get("norm.out", residual.shape, ctx.dtype)
        ops.norm_add(branch, residual, self.weight, self.eps, self.plus_one, mult, next_weight=then.weight,
                     next_eps=then.eps, next_plus_one=then.plus_one, next_out=out)
        return out


class PendingBranch:
    """A sublayer's output that has not joined the residual streams yet, with the connection
    weights it joins them by: ``x_t <- sum_s mix[s, t] x_s + out[t] y``.  A hyper-connected block
    hands it on where other blocks hand on a plain branch output; the next :class:`HyperNorm`
    (the next sublayer's, the next layer's or the model's last norm) folds it in."""

    __slots__ = ("y", "mix", "out")

    def __init__(self, y: torch.Tensor, mix: torch.Tensor, out: torch.Tensor):
        self.y, self.mix, self.out = y, mix, out


@register_norm("hyper_norm")
class HyperNorm(Norm):
    """The norm in front of a sublayer of a model with several residual streams
    (hyper-connections).  The residual is ``[T, streams, H]`` float32; the sublayer reads ``u =
    sum_s in[s] x_s``, normed here, and its output ``y`` later joins every stream: ``x_t <- sum_s
    mix[s, t] x_s + out[t] y`` (``mix`` is indexed ``[from, to]``).  One launch folds in the branch
    that is still pending, forms ``u`` and norms it.

    params: ``size``, ``eps``, ``streams``, ``tensor`` (the norm weight's name below the prefix),
    ``bias_tensor`` (None: no bias), ``center`` (default True: layer norm - the mean is taken off and
    the variance is the mean of the squared deviations; False: RMS norm), ``connection`` (the prefix
    of the ``in``, ``out`` and ``mix`` tensors below the layer's; None: the norm reads the plain sum
    of the streams and no branch leaves through it - the model's last norm; ``"identity"``: no
    tensors, every weight is one - with one stream the plain pre-norm residual ``x <- x + y``)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.size = int(p["size"])
        self.eps = float(p["eps"])
        self.streams = int(p.get("streams", 1))
        self.center = bool(p.get("center", True))
        self.weight_name = self.name(p["tensor"])
        self.bias_name = self.name(p["bias_tensor"]) if p.get("bias_tensor") else None
        conn = p.get("connection")
        self.identity = conn == "identity"
        if self.identity and self.streams != 1:
            raise ValueError("connection weights of one are the plain residual: they need streams = 1")
        self.conn = {k: self.name(f"{conn}.{k}") for k in ("in", "out", "mix")} if conn and not self.identity else None
        self.weight = self.bias = self.w_in = self.w_out = self.w_mix = None

    def tensor_specs(self) -> List[TensorSpec]:
        S = self.streams
        specs = [TensorSpec(self.weight_name, (self.size,), role="small32", init=Init(mean=1.0, std=0.0), tag="norm")]
        if self.bias_name:
            specs.append(TensorSpec(self.bias_name, (self.size,), role="small32", init=Init(0.0, 0.02), tag="bias"))
        if self.conn:
            # near the plain residual sum: every stream keeps itself, reads and writes are spread evenly
            specs += [TensorSpec(self.conn["in"], (S,), role="small32", init=Init(1.0 / S, 0.1 / S), tag="connection"),
                      TensorSpec(self.conn["out"], (S,), role="small32", init=Init(1.0, 0.1), tag="connection"),
                      TensorSpec(self.conn["mix"], (S, S), role="small32", init=Init(0.0, 0.1 / S, eye=1.0), tag="connection_mix")]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]
        self.bias = tensors[self.bias_name] if self.bias_name else None
        if self.conn:
            self.w_in, self.w_out, self.w_mix = (tensors[self.conn[k]] for k in ("in", "out", "mix"))
        elif self.identity:
            ones = torch.ones(1, dtype=torch.float32, device=self.weight.device)
            self.w_in, self.w_out, self.w_mix = ones, ones, ones.view(1, 1)

    def libraries(self, dtype) -> List[str]:
        return ["rowwise"]

    def pending(self, y: torch.Tensor) -> PendingBranch:
        """``y`` (this norm's sublayer's output) with the weights it joins the streams by."""
        if not self.conn and not self.identity:
            raise ValueError("a norm without connection weights has no sublayer whose output could leave through it")
        return PendingBranch(y, self.w_mix, self.w_out)

    def forward(self, ctx: StepContext, delta, residual: torch.Tensor) -> torch.Tensor:
        if residual.dim() == 2 and self.streams == 1:
            residual = residual.unsqueeze(1)          # one stream: the plain residual [T, H]
        if residual.dim() != 3 or residual.shape[1] != self.streams:
            raise ValueError(f"hyper_norm: the residual must be [T, {self.streams}, H]")
        if delta is not None and not isinstance(delta, PendingBranch):
            raise ValueError("hyper_norm: a branch reaches the streams through its connection weights "
                             "(PendingBranch), not as a plain tensor")
        T, _, H = residual.shape
        out = ctx.workspace.get("norm.out", (T, H), ctx.dtype)
        y, mix, w_out = (delta.y, delta.mix, delta.out) if delta is not None else (None, None, None)
        ops.hyper_norm(residual, y, mix, w_out, self.w_in, self.weight, self.bias, self.eps, self.center, out)
        return out
