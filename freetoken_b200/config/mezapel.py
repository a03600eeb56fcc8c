"""Typed configuration of the Mezapel decoder, read from ``config.json``.

A Mezapel model embeds a token as ``E[token] * scale`` plus a row of a second table picked by a
hash of the token and the one before it, runs pre-norm layers (layer norm with weight and bias)
over one residual stream or over ``streams`` copies joined by hyper-connections::

    u = sum_s in[s] x_s;   y = sublayer(layernorm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y

and ends in a layer norm and a head.  A range of layers may run several times in a row with the
same weights (``loop``), each pass with a cache of its own.  Mixers, both grouped-query softmax
attention with a sigmoid gate read from the mixer's input:

* ``attention``: RMS norm over the whole q and the whole k projection, the first ``rot.dims``
  dimensions of a head rotated in halves with YaRN-scaled frequencies, a mask in chunks of
  ``mask.size`` positions, softmax weights ``e^s / (1 + sum e^s)`` (a sink of score 0), one gate
  per head;
* ``attention_2``: a causal convolution of ``conv`` taps behind each of q, k and v, RMS norm per
  head with a weight the heads share, Llama-3.1-scaled frequencies, scores capped by ``softcap *
  tanh(s / softcap)``, a sliding window of ``mask.size`` keys, a learned sink per head, one gate per
  output value.

Feed-forward: ``W_down (silu(W_gate h) (W_up h))`` or none.

config.json keys: ``architecture`` (``"Mezapel"``), ``vocab``, ``width``, ``streams`` (absent: the plain
residual), ``norm.eps``, ``embedding.{scale, bigram.{buckets, mul_prev, mul_cur}}``, ``loop.{start, stop,
times}`` and ``layers[i]`` with ``type``, ``mixer`` and ``mlp``.  Mixer keys: ``heads, kv_heads, dim, vdim,
scale, mask.size, rot.{base, dims, scaling}``; ``attention_2`` also ``conv`` and ``softcap``.  ``rot.scaling``
- ``attention``: ``factor, original, fast, slow``; ``attention_2``: ``factor, original, low, high``.  mlp keys:
``kind`` (``dense``), ``ff``.  Tensors: ``embed``, ``bigram``, ``final.norm[.b]``, ``head`` and ``l<i>.{norm1[.b],
norm2[.b], hc1.*, hc2.*, mix.*, mlp.*}``.  The reference has no model of this design; the module
follows the shape of python/freetoken/models/minimax_m3/args.py:135-254.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .model_plan import ConfigError, LayerSpec, ModelPlan, PartSpec, RunEntry

ARCHITECTURE = "Mezapel"
MIXER_TYPES = ("attention", "attention_2")
MLP_KINDS = ("dense",)
# constants the design fixes
ZERO_SINK_SCORE = 0.0            # a denominator of 1 + sum(e^s) is that of a sink with the score 0
SCALING_OF = {"attention": "yarn", "attention_2": "llama3"}     # which rule a mixer's rot.scaling follows
SCALING_KEYS = {"yarn": ("factor", "original", "fast", "slow"), "llama3": ("factor", "original", "low", "high")}
MAX_STREAMS = 8                  # what the stream kernel keeps in registers
NO_POSITION_LIMIT = 1 << 30      # rotation angles are computed, not tabulated by the design


@dataclass(frozen=True)
class MezapelMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask: int                                   # chunk size (attention) or window (attention_2); 0: all keys
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[Tuple[Tuple[str, float], ...]]     # sorted (key, value) pairs incl. kind, or None
    conv: int = 0
    softcap: float = 0.0


@dataclass(frozen=True)
class MezapelLayer:
    type: str
    mixer: MezapelMixer
    ff: Optional[int]                           # width of the dense feed-forward's middle, None: no feed-forward


@dataclass(frozen=True)
class Bigram:
    buckets: int
    mul_prev: int
    mul_cur: int


def _need(d: Any, key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    return d[key]


def _positive(where: str, **values) -> None:
    for name, v in values.items():
        if not v > 0:
            raise ConfigError(f"config.json: '{where}{name}' must be positive")


def _read_mixer(kind: str, m: Any, where: str) -> MezapelMixer:
    heads, dim = int(_need(m, "heads", where)), int(_need(m, "dim", where))
    kv_heads, vdim = int(m.get("kv_heads") or heads), int(m.get("vdim") or dim)
    _positive(where, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim)
    if heads % kv_heads:
        raise ConfigError(f"config.json: '{where}kv_heads' = {kv_heads} does not divide heads = {heads}")
    if max(dim, vdim) > 1024:
        raise ConfigError(f"config.json: '{where}dim' / 'vdim' above 1024 is not supported")
    rot = m.get("rot") or {}
    rot_dims = int(rot.get("dims") or 0)
    rot_base = float(rot.get("base") or 1.0)
    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"config.json: '{where}rot.dims' = {rot_dims} must be even and at most dim = {dim}")
    if rot_dims and not rot_base > 1.0:
        raise ConfigError(f"config.json: '{where}rot.base' must be above 1")
    scaling = None
    if rot_dims and rot.get("scaling"):
        rule = SCALING_OF[kind]
        values = {"kind": rule}
        for key in SCALING_KEYS[rule]:
            values[key] = float(_need(rot["scaling"], key, where + "rot.scaling."))
        _positive(where + "rot.scaling.", factor=values["factor"], original=values["original"])
        if rule == "yarn":
            _positive(where + "rot.scaling.", fast=values["fast"], slow=values["slow"])
        else:
            _positive(where + "rot.scaling.", low=values["low"], high=values["high"])
        scaling = tuple(sorted(values.items(), key=lambda kv: kv[0]))
    mask = int((m.get("mask") or {}).get("size") or 0)
    if mask < 0:
        raise ConfigError(f"config.json: '{where}mask.size' must not be negative")
    conv = int(m.get("conv") or 0) if kind == "attention_2" else 0
    softcap = float(m.get("softcap") or 0.0) if kind == "attention_2" else 0.0
    if conv < 0 or softcap < 0:
        raise ConfigError(f"config.json: '{where}conv' and 'softcap' must not be negative")
    return MezapelMixer(heads, kv_heads, dim, vdim, float(_need(m, "scale", where)), mask, rot_base, rot_dims,
                        scaling, conv, softcap)


@dataclass(frozen=True)
class MezapelConfig:
    vocab: int
    width: int
    streams: int                 # 0: one plain residual stream without connection weights
    norm_eps: float
    embed_scale: float
    bigram: Optional[Bigram]
    layers: Tuple[MezapelLayer, ...]
    loop: Optional[Tuple[int, int, int]]        # (start, stop, times)
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MezapelConfig":
        listed = _need(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[MezapelLayer] = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]."
            kind = str(_need(entry, "type", where))
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not one of {list(MIXER_TYPES)}")
            mixer = _read_mixer(kind, _need(entry, "mixer", where), where + "mixer.")
            ff = None
            mlp = entry.get("mlp")
            if mlp:
                mlp_kind = str(mlp.get("kind", "dense"))
                if mlp_kind not in MLP_KINDS:
                    raise ConfigError(f"config.json: '{where}mlp.kind' = {mlp_kind!r} is not one of {list(MLP_KINDS)}")
                ff = int(_need(mlp, "ff", where + "mlp."))
                _positive(where + "mlp.", ff=ff)
            layers.append(MezapelLayer(kind, mixer, ff))
        emb = raw.get("embedding") or {}
        bigram = None
        if emb.get("bigram"):
            b = emb["bigram"]
            bigram = Bigram(int(_need(b, "buckets", "embedding.bigram.")), int(_need(b, "mul_prev", "embedding.bigram.")),
                            int(_need(b, "mul_cur", "embedding.bigram.")))
            _positive("embedding.bigram.", buckets=bigram.buckets)
            if bigram.mul_prev < 0 or bigram.mul_cur < 0:
                raise ConfigError("config.json: 'embedding.bigram.mul_prev' and 'mul_cur' must not be negative")
        loop = None
        if raw.get("loop"):
            lp = raw["loop"]
            loop = (int(_need(lp, "start", "loop.")), int(_need(lp, "stop", "loop.")), int(lp.get("times", 1)))
            if not 0 <= loop[0] <= loop[1] <= len(layers) or loop[2] < 1:
                raise ConfigError(f"config.json: 'loop' = {dict(lp)} must satisfy 0 <= start <= stop <= "
                                  f"{len(layers)} layers and times >= 1")
        streams = raw.get("streams")
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  streams=int(streams) if streams is not None else 0,
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")),
                  embed_scale=float(emb["scale"]) if emb.get("scale") is not None else 1.0, bigram=bigram,
                  layers=tuple(layers), loop=loop, raw=dict(raw))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if streams is not None and not 1 <= cfg.streams <= MAX_STREAMS:
            raise ConfigError(f"config.json: 'streams' = {cfg.streams} must lie in 1..{MAX_STREAMS}")
        if cfg.norm_eps < 0:
            raise ConfigError("config.json: 'norm.eps' must not be negative")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    def run_order(self) -> List[int]:
        """Layer indices in the order they run: the looped range repeats as a whole."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def _mixer_spec(cfg: MezapelConfig, layer: MezapelLayer) -> PartSpec:
    m = layer.mixer
    position = PartSpec("rotary_neox", {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                        "max_position": NO_POSITION_LIMIT, "exact_angles": True,
                                        "scaling": dict(m.rot_scaling) if m.rot_scaling else None})
    params: Dict[str, Any] = {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
        "value_dim": m.vdim, "sm_scale": m.scale, "qk_norm_eps": cfg.norm_eps, "position": position, "scope": "mix",
        "fill_heads": True,
        "checkpoint_names": {"q": "q", "k": "k", "v": "v", "o": "o", "qkv": "qkvg", "q_norm": "q.norm",
                             "k_norm": "k.norm", "gate": "g", "sink": "sink", "q_conv": "q.conv",
                             "k_conv": "k.conv", "v_conv": "v.conv", "qkv_conv": "qkv.conv"}}
    if layer.type == "attention":
        params.update(qk_norm="per_layer", chunk=m.mask or None, sink_value=ZERO_SINK_SCORE, gate="head")
    else:
        params.update(qk_norm="per_head", sliding_window=m.mask or None, softcap=m.softcap or None, sink=True,
                      gate="element", conv_taps=m.conv)
    return PartSpec("paged_attention", params)


def build_plan(cfg: MezapelConfig) -> ModelPlan:
    W, S = cfg.width, max(cfg.streams, 1)

    def norm(tensor: str, connection: Optional[str]) -> PartSpec:
        return PartSpec("hyper_norm", {"size": W, "eps": cfg.norm_eps, "streams": S, "tensor": tensor,
                                       "bias_tensor": tensor + ".b", "center": True,
                                       "connection": connection if (cfg.streams or connection is None) else "identity"})

    layers: List[LayerSpec] = []
    for i, layer in enumerate(cfg.layers):
        ffn = None
        if layer.ff is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": W, "intermediate_size": layer.ff, "activation": "silu",
                                         "gated": True, "scope": "mlp",
                                         "names": {"gate": "gate", "up": "up", "down": "down", "gate_up": "gate_up"}})
        layers.append(LayerSpec(
            prefix=f"l{i}", block=PartSpec("hyper", {}), mixer=_mixer_spec(cfg, layer), feed_forward=ffn,
            mixer_norm=norm("norm1", "hc1"), feed_forward_norm=norm("norm2", "hc2") if ffn is not None else None))
    embedding = {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "", "tensor": "embed", "scale": cfg.embed_scale}
    if cfg.bigram is not None:
        embedding.update(pair_tensor="bigram", buckets=cfg.bigram.buckets, mul_prev=cfg.bigram.mul_prev,
                         mul_cur=cfg.bigram.mul_cur)
    plan = ModelPlan(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", embedding),
        layers=tuple(layers), schedule=tuple(RunEntry(i) for i in cfg.run_order()),
        final_norm=PartSpec("hyper_norm", {**norm("final.norm", None).params, "prefix": ""}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "", "tensor": "head",
                                  "tied_to": None}),
        max_position=NO_POSITION_LIMIT, residual_streams=S)
    plan.validate()
    return plan
