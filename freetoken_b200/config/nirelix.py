"""Typed configuration of the Nirelix decoder, read from ``config.json``.

A Nirelix model keeps ``streams`` copies of the residual stream (hyper-connections).  A sublayer
reads a weighted sum of the streams, layer-normed with weight and bias, and its output joins every
stream again through a small mixing matrix::

    u = sum_s in[s] x_s;   y = sublayer(layernorm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y

A layer is a mixer sublayer and, unless its ``mlp`` is null, a feed-forward sublayer.  Mixers:

* ``retention``: per head ``S <- c_h S + k v^T``, ``o = S^T q`` with a constant decay ``c_h`` from the
  config, q and k rotated in halves, k times ``dim^-1/2``; the read-out is RMS-normed per head
  without a weight, gated by ``silu(W_g h)``;
* ``channel_delta``: the gated delta rule behind short convolutions, with a decay per head AND key
  channel, ``exp(-exp(A_h) softplus(W_a2 W_a1 h + dt_bias))``, a read-out norm whose weight the heads
  share, and a gate ``sigmoid(W_g2 W_g1 h)``.  The width of the middle of the two-step projections
  is the one size config.json does not state: it is read from the checkpoint's tensor shapes
  (:func:`sizes_from_tensors`), or given as ``mixer.low_rank`` (and ``mixer.gate_rank`` where the gate's
  middle has another width than the decay's) for a model without a checkpoint;
* ``latent_attention``: queries through a normed latent, keys and values made from a normed latent
  of ``kv_rank`` values plus ``rot_dim`` rotated key values shared by the heads (pairs ``(2i, 2i + 1)``),
  softmax inside a sliding window, a sigmoid gate per output value.

Feed-forwards: ``dense`` - ``min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, +-L) + 1)``; ``moe`` - experts
``silu(W_gate h) (W_up h)`` chosen by ``sigmoid(router) + correction`` inside the ``groups.keep`` best of
``groups.count`` groups of neighbours (a group's value: its two largest choice scores), weighted by
the uncorrected scores, normalised and times ``router.scale``.

config.json keys: ``architecture`` (``"Nirelix"``), ``vocab``, ``width``, ``streams``, ``norm.eps`` and
``layers[i]`` with ``type``, ``mixer`` and ``mlp``.  Mixer keys - retention: ``heads, dim, vdim, decay,
rot.{base, dims}``; channel_delta: ``heads, kv_heads, dim, vdim, conv``; latent_attention: ``heads, dim,
rot_dim, vdim, q_rank, kv_rank, scale, mask.size, rot.{base, dims}``.  mlp keys: ``kind`` (``dense``: ``ff,
limit``; ``moe``: ``expert.ff``, ``router.{experts, top, scale, groups.{count, keep}}``).  Tensors: ``embed``,
``final.norm[.b]``, ``head`` and ``l<i>.{norm1[.b], norm2[.b], hc1.*, hc2.*, mix.*, mlp.*}``.  The reference
has no model of this design; the module follows the shape of
python/freetoken/models/minimax_m3/args.py:135-254.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .model_plan import ConfigError, LayerSpec, ModelPlan, PartSpec, RunEntry

ARCHITECTURE = "Nirelix"
MIXER_TYPES = ("retention", "channel_delta", "latent_attention")
MLP_KINDS = ("dense", "moe")
# constants the design fixes
DENSE_GATE_ALPHA = 1.702         # g * sigmoid(alpha * g) in the dense feed-forward
UNIT_NORM_EPS = 1e-6             # under the root of the delta rule's unit norms
MAX_STREAMS = 8                  # what the stream kernel keeps in registers
NO_POSITION_LIMIT = 1 << 30      # rotation angles are computed, not tabulated by the design


@dataclass(frozen=True)
class RetentionMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class ChannelDeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    low_rank: int
    gate_rank: int


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: int
    rot_base: float


@dataclass(frozen=True)
class NirelixMLP:
    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    groups: int = 1
    keep: int = 1


@dataclass(frozen=True)
class NirelixLayer:
    type: str
    mixer: Any
    mlp: Optional[NirelixMLP]


def _need(d: Any, key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    return d[key]


def _positive(where: str, **values: int) -> None:
    for name, v in values.items():
        if v <= 0:
            raise ConfigError(f"config.json: '{where}{name}' must be positive")


def _rot(m: Any, where: str, limit: int) -> Tuple[float, int]:
    rot = _need(m, "rot", where)
    base, dims = float(_need(rot, "base", where + "rot.")), int(_need(rot, "dims", where + "rot."))
    if dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"config.json: '{where}rot.dims' = {dims} must be even and at most {limit}")
    if dims and base <= 0:
        raise ConfigError(f"config.json: '{where}rot.base' must be positive")
    return base, dims


def _read_retention(m: Any, where: str) -> RetentionMixer:
    heads, dim = int(_need(m, "heads", where)), int(_need(m, "dim", where))
    vdim = int(m.get("vdim") or dim)
    _positive(where, heads=heads, dim=dim, vdim=vdim)
    decay = tuple(float(v) for v in _need(m, "decay", where))
    if len(decay) != heads:
        raise ConfigError(f"config.json: '{where}decay' lists {len(decay)} values for {heads} heads")
    if dim > 256:
        raise ConfigError(f"config.json: '{where}dim' above 256 is not supported")
    base, dims = _rot(m, where, dim)
    return RetentionMixer(heads, dim, vdim, decay, base, dims)


def _read_channel_delta(m: Any, where: str) -> ChannelDeltaMixer:
    d = ChannelDeltaMixer(heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]),
                          dim=int(_need(m, "dim", where)), vdim=int(m.get("vdim") or m["dim"]),
                          conv=int(_need(m, "conv", where)), low_rank=int(m.get("low_rank") or 0),
                          gate_rank=int(m.get("gate_rank") or m.get("low_rank") or 0))
    _positive(where, heads=d.heads, kv_heads=d.kv_heads, dim=d.dim, vdim=d.vdim, conv=d.conv)
    if d.heads % d.kv_heads:
        raise ConfigError(f"config.json: '{where}kv_heads' = {d.kv_heads} does not divide heads = {d.heads}")
    if d.dim > 256:
        raise ConfigError(f"config.json: '{where}dim' above 256 is not supported")
    if d.low_rank <= 0:
        raise ConfigError(f"config.json: '{where}low_rank' is neither given nor known from the checkpoint's "
                          f"tensor shapes (the width of the middle of the decay's two-step projection)")
    return d


def _read_latent(m: Any, where: str) -> LatentMixer:
    rot_dim = int(m.get("rot_dim") or 0)
    base, dims = _rot(m, where, max(rot_dim, 0)) if rot_dim else (1.0, 0)
    if rot_dim and dims != rot_dim:
        raise ConfigError(f"config.json: '{where}rot.dims' = {dims} must equal rot_dim = {rot_dim}")
    a = LatentMixer(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)), rot_dim=rot_dim,
                    vdim=int(m.get("vdim") or m["dim"]), q_rank=int(_need(m, "q_rank", where)),
                    kv_rank=int(_need(m, "kv_rank", where)), scale=float(_need(m, "scale", where)),
                    window=int(_need(_need(m, "mask", where), "size", where + "mask.")), rot_base=base)
    _positive(where, heads=a.heads, dim=a.dim, vdim=a.vdim, q_rank=a.q_rank, kv_rank=a.kv_rank)
    _positive(where + "mask.", size=a.window)
    if a.kv_rank + a.rot_dim > 1024:
        raise ConfigError(f"config.json: '{where}kv_rank' + rot_dim above 1024 is not supported")
    return a


_READERS = {"retention": _read_retention, "channel_delta": _read_channel_delta, "latent_attention": _read_latent}


def _read_mlp(mlp: Any, where: str) -> Optional[NirelixMLP]:
    if not mlp:
        return None
    kind = str(mlp.get("kind", "dense"))
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: '{where}kind' = {kind!r} is not one of {list(MLP_KINDS)}")
    if kind == "dense":
        out = NirelixMLP("dense", int(_need(mlp, "ff", where)), limit=float(_need(mlp, "limit", where)))
        _positive(where, ff=out.ff)
        if not out.limit > 0:
            raise ConfigError(f"config.json: '{where}limit' must be positive")
        return out
    expert, router = _need(mlp, "expert", where), _need(mlp, "router", where)
    groups = router.get("groups") or {}
    out = NirelixMLP("moe", int(_need(expert, "ff", where + "expert.")),
                     experts=int(_need(router, "experts", where + "router.")),
                     top=int(_need(router, "top", where + "router.")), scale=float(router.get("scale", 1.0)),
                     groups=int(groups.get("count", 1)), keep=int(groups.get("keep", groups.get("count", 1))))
    _positive(where, ff=out.ff, experts=out.experts, top=out.top, groups=out.groups, keep=out.keep)
    if out.top > out.experts:
        raise ConfigError(f"config.json: '{where}router.top' = {out.top} exceeds experts = {out.experts}")
    if out.experts % out.groups or out.keep > out.groups or out.groups > 256:
        raise ConfigError(f"config.json: '{where}router.groups' = {out.groups} (keep {out.keep}) must divide "
                          f"experts = {out.experts}, keep at most count, count at most 256")
    if out.keep * (out.experts // out.groups) < out.top:
        raise ConfigError(f"config.json: '{where}router.top' = {out.top} experts do not fit into "
                          f"{out.keep} groups of {out.experts // out.groups}")
    return out


@dataclass(frozen=True)
class NirelixConfig:
    vocab: int
    width: int
    streams: int
    norm_eps: float
    layers: Tuple[NirelixLayer, ...]
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NirelixConfig":
        listed = _need(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[NirelixLayer] = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]."
            kind = str(_need(entry, "type", where))
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not one of {list(MIXER_TYPES)}")
            mixer = _READERS[kind](_need(entry, "mixer", where), where + "mixer.")
            layers.append(NirelixLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + "mlp.")))
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  streams=int(raw.get("streams", 1)),
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")), layers=tuple(layers), raw=dict(raw))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not 1 <= cfg.streams <= MAX_STREAMS:
            raise ConfigError(f"config.json: 'streams' = {cfg.streams} must lie in 1..{MAX_STREAMS}")
        if cfg.norm_eps < 0:
            raise ConfigError("config.json: 'norm.eps' must not be negative")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)


def sizes_from_tensors(raw: Mapping[str, Any], shapes: Mapping[str, Tuple[int, ...]]) -> Dict[str, Any]:
    """``raw`` with the sizes that only the checkpoint states filled in: the widths of the middles of a
    ``channel_delta`` mixer's two-step projections are the numbers of rows of ``l<i>.mix.a1`` (decay)
    and ``l<i>.mix.g1`` (gate)."""
    out = dict(raw)
    layers = []
    for i, entry in enumerate(raw.get("layers") or []):
        if isinstance(entry, Mapping) and entry.get("type") == "channel_delta" and isinstance(entry.get("mixer"), Mapping):
            for key, tensor in (("low_rank", "a1"), ("gate_rank", "g1")):
                shape = shapes.get(f"l{i}.mix.{tensor}")
                if shape and not entry["mixer"].get(key):
                    entry = {**entry, "mixer": {**entry["mixer"], key: int(shape[0])}}
        layers.append(entry)
    out["layers"] = layers
    return out


def _mixer_spec(cfg: NirelixConfig, layer: NirelixLayer) -> PartSpec:
    W, m = cfg.width, layer.mixer
    if layer.type == "retention":
        return PartSpec("retention", {
            "hidden_size": W, "heads": m.heads, "key_dim": m.dim, "head_dim": m.vdim, "decay": m.decay,
            "norm_eps": cfg.norm_eps, "scope": "mix",
            "position": PartSpec("rotary_neox", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                                 "max_position": NO_POSITION_LIMIT, "exact_angles": True}),
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "in": "qkvg"}})
    if layer.type == "channel_delta":
        return PartSpec("channel_delta", {
            "hidden_size": W, "heads": m.heads, "key_heads": m.kv_heads, "key_dim": m.dim, "head_dim": m.vdim,
            "conv_taps": m.conv, "low_rank": m.low_rank, "gate_rank": m.gate_rank, "norm_eps": cfg.norm_eps, "unit_eps": UNIT_NORM_EPS,
            "scope": "mix",
            "names": {"q": "q", "k": "k", "v": "v", "beta": "b", "decay_down": "a1", "decay_up": "a2",
                      "gate_down": "g1", "gate_up": "g2", "q_conv": "q.conv", "k_conv": "k.conv",
                      "v_conv": "v.conv", "a_log": "A_log", "dt_bias": "dt_bias", "norm": "norm", "o": "o",
                      "in": "qkvagb", "conv": "qkv.conv"}})
    return PartSpec("latent_attention", {
        "hidden_size": W, "num_heads": m.heads, "qk_dim": m.dim, "v_dim": m.vdim, "rank": m.kv_rank,
        "sm_scale": m.scale, "norm_eps": cfg.norm_eps, "output_gate": True, "gate_per": "element",
        "q_rank": m.q_rank, "rot_dim": m.rot_dim, "sliding_window": m.window, "scope": "mix",
        "position": PartSpec("rotary_interleaved", {"head_dim": max(m.rot_dim, 2), "rotary_dim": m.rot_dim,
                                                    "theta": m.rot_base, "max_position": NO_POSITION_LIMIT,
                                                    "exact_angles": True}),
        "names": {"q": "q", "q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "down": "dkv",
                  "latent_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "o": "o", "in": "dqkvg"}})


def _mlp_spec(cfg: NirelixConfig, mlp: NirelixMLP) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff,
                                      "activation": "swigluoai", "act_alpha": DENSE_GATE_ALPHA,
                                      "act_limit": mlp.limit, "gated": True, "scope": "mlp",
                                      "names": {"gate": "gate", "up": "up", "down": "down", "gate_up": "gate_up"}})
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "intermediate_size": mlp.ff, "num_experts": mlp.experts, "top_k": mlp.top,
        "scoring": "sigmoid", "use_bias": True, "renormalize": True, "scale": mlp.scale,
        "groups": mlp.groups, "keep_groups": mlp.keep, "activation": "silu", "scope": "mlp",
        "checkpoint_names": {"router": "router", "bias": "correction", "gate_up": "experts.gate_up",
                             "down": "experts.down", "gate": "e{e}.gate", "up": "e{e}.up",
                             "down_each": "e{e}.down"}})


def build_plan(cfg: NirelixConfig) -> ModelPlan:
    W, S = cfg.width, cfg.streams

    def norm(tensor: str, connection: Optional[str]) -> PartSpec:
        return PartSpec("hyper_norm", {"size": W, "eps": cfg.norm_eps, "streams": S, "tensor": tensor,
                                       "bias_tensor": tensor + ".b", "center": True, "connection": connection})

    layers: List[LayerSpec] = []
    for i, layer in enumerate(cfg.layers):
        ffn = _mlp_spec(cfg, layer.mlp) if layer.mlp is not None else None
        layers.append(LayerSpec(
            prefix=f"l{i}", block=PartSpec("hyper", {}), mixer=_mixer_spec(cfg, layer), feed_forward=ffn,
            mixer_norm=norm("norm1", "hc1"), feed_forward_norm=norm("norm2", "hc2") if ffn is not None else None))
    plan = ModelPlan(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "",
                                               "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("hyper_norm", {**norm("final.norm", None).params, "prefix": ""}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "", "tensor": "head",
                                  "tied_to": None}),
        max_position=NO_POSITION_LIMIT, residual_streams=S)
    plan.validate()
    return plan
