"""Pofazen: a small decoder whose ``config.json`` lists its layers one by one.
Its typed configuration, its layer plan and its entry in the architecture
registry; everything this engine knows about the design by name is here.

The design, as this file builds it from the parts:

* embedding rows, RMS-normed with ``embed.norm``;
* every layer is a *postnorm* block: the residual stream itself is normed
  after each sum, ``x <- norm1(alpha x + mixer(x))`` and ``x <- norm2(alpha x +
  ff(x))`` with ``alpha = postln_alpha``, and the sublayers read x as it is;
* mixer ``parallel``: two mixers side by side on the same input, their
  results scaled (``left_scale``, ``right_scale``) and added.  Left:
  grouped-query attention without biases, q and k heads RMS-normed (one weight
  for q, one for k), the first ``rot.dims`` entries of a head rotated in
  interleaved pairs with frequencies rescaled in three bands, an explicit
  score scale, a sliding window that also keeps the first ``mask.keep_first``
  positions visible, and a sigmoid gate on the concatenated heads.  Right: the
  gated delta rule behind a short causal convolution (``parts/recurrent.py``);
* mixer ``wkv``: token-shift mixes, a per-channel decay from a low-rank
  product, a bonus for the current token (``parts/recurrent.py``).  The rank of
  the decay's product is the shape of ``w1`` in the model file (``decay_rank``
  in the mixer's configuration where there is no file);
* feed-forward ``dense``: ``down(silu(gate(x)) * up(x))``;
* final RMS norm (``final.norm``) and an untied linear head (``head``).

The design puts no limit on positions; block tables need a width, so
``max_positions`` (an engine knob, default 131072) may be given in the file.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.model_config import ConfigError
from ..model_registry import register_architecture
from ..parts.base import PartSpec
from .decoder import ModelSpec

ARCHITECTURE = "Pofazen"
DEFAULT_MAX_POSITIONS = 131072
UNIT_EPS = 1e-6            # the design fixes it: q and k of the delta rule are x / sqrt(sum x^2 + 1e-6)


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = int(_need(d, key, where))
    if v < 1:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]             # None: every earlier key
    keep_first: int
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[Tuple[float, float, float, float]]     # factor, low, high, original


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: GatedDeltaConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class WKVConfig:
    heads: int
    dim: int
    decay_rank: int


@dataclass(frozen=True)
class PofazenLayer:
    type: str                         # "parallel" | "wkv"
    mixer: object
    ff: Optional[int]                 # hidden size of the feed-forward (None: the layer has none)


def _heads(mx, where):
    heads = _pos_int(mx, "heads", where)
    kvh = int(mx.get("kv_heads") or heads)
    if kvh < 1 or heads % kvh:
        raise ConfigError(f"config.json: {where}: heads ({heads}) not divisible by kv_heads ({kvh})")
    return heads, kvh


def _left(mx, where) -> WindowAttentionConfig:
    heads, kvh = _heads(mx, where)
    dim = _pos_int(mx, "dim", where)
    mask = mx.get("mask") or {}
    window = None if mask.get("size") is None else _pos_int(mask, "size", where + ".mask")
    keep = int(mask.get("keep_first") or 0)
    if keep < 0:
        raise ConfigError(f"config.json: {where}.mask.keep_first must not be negative")
    rot = mx.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    if dims % 2 or not 0 <= dims <= dim:
        raise ConfigError(f"config.json: {where}.rot.dims = {dims}: must be even and at most dim ({dim})")
    sc = rot.get("scaling")
    scaling = None
    if sc:
        scaling = tuple(float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "low", "high", "original"))
    return WindowAttentionConfig(heads, kvh, dim, int(mx.get("vdim") or dim), float(_need(mx, "scale", where)), window,
                                 keep if window is not None else 0, dims, float(rot.get("base", 10000.0)), scaling)


def _right(mx, where) -> GatedDeltaConfig:
    heads, kvh = _heads(mx, where)
    return GatedDeltaConfig(heads, kvh, _pos_int(mx, "dim", where), _pos_int(mx, "vdim", where), _pos_int(mx, "conv", where))


@dataclass(frozen=True)
class PofazenConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    layers: Tuple[PofazenLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict, tensor_shapes: Optional[dict] = None) -> "PofazenConfig":
        vocab, width = _pos_int(raw, "vocab", "the model"), _pos_int(raw, "width", "the model")
        eps = float(_need(_need(raw, "norm", "the model"), "eps", "norm"))
        alpha = float(_need(raw, "postln_alpha", "the model"))
        layers_raw = _need(raw, "layers", "the model")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind, mx = _need(lr, "type", where), _need(lr, "mixer", where)
            mw = where + ".mixer"
            if kind == "parallel":
                mixer = ParallelMixerConfig(_left(_need(mx, "left", mw), mw + ".left"), _right(_need(mx, "right", mw), mw + ".right"),
                                            float(_need(mx, "left_scale", mw)), float(_need(mx, "right_scale", mw)))
            elif kind == "wkv":
                rank = mx.get("decay_rank")
                if tensor_shapes is not None:
                    shape = tensor_shapes.get(f"l{i}.mix.w1")
                    if shape is None or len(shape) != 2:
                        raise ConfigError(f"the model file has no matrix 'l{i}.mix.w1', whose rows are the decay's rank")
                    rank = shape[0]
                if rank is None:
                    raise ConfigError(f"config.json: {mw} has no 'decay_rank' (without a model file nothing else gives it)")
                mixer = WKVConfig(_pos_int(mx, "heads", mw), _pos_int(mx, "dim", mw), int(rank))
            else:
                raise ConfigError(f"config.json: {where}.type = {kind!r}: this design has 'parallel' and 'wkv' mixers")
            mlp = lr.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind = {mlp.get('kind')!r}: only 'dense' is computed")
                ff = _pos_int(mlp, "ff", where + ".mlp")
            layers.append(PofazenLayer(kind, mixer, ff))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab, width, eps, alpha, tuple(layers), int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS), eos)


def pofazen_spec(cfg: PofazenConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda tensor, prefix="", optional=False: PartSpec(
        "rmsnorm", dict(width=W, eps=cfg.eps, tensor=tensor, optional=optional), prefix=prefix)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "parallel":
            l, r = m.left, m.right
            left = PartSpec("gqa_attention", dict(
                hidden_size=W, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim, v_head_dim=l.vdim,
                qkv_bias=False, o_bias=False, scale=l.scale, window=l.window, keep_first=l.keep_first,
                qk_norm_eps=cfg.eps, gate=True,
                position=PartSpec("rotary_scaled", dict(
                    rotary_dim=l.rot_dims, theta=l.rot_base, interleaved=True,
                    scaling=None if l.rot_scaling is None else dict(zip(("factor", "low", "high", "original"), l.rot_scaling)))),
                names=dict(q="q", k="k", v="v", o="o", g="g", q_norm="q.norm", k_norm="k.norm")), prefix=p + "mix.left.")
            right = PartSpec("gated_delta", dict(
                hidden_size=W, num_heads=r.heads, num_kv_heads=r.kv_heads, head_dim=r.dim, v_head_dim=r.vdim,
                conv=r.conv, eps=cfg.eps, unit_eps=UNIT_EPS,
                names=dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", b="b", a="a",
                           A_log="A_log", dt_bias="dt_bias", g="g", norm="norm", o="o")), prefix=p + "mix.right.")
            mixer = PartSpec("sum", dict(mixers=[left, right], scales=[m.left_scale, m.right_scale]), prefix=p + "mix.")
        else:
            mixer = PartSpec("wkv", dict(hidden_size=W, num_heads=m.heads, head_dim=m.dim, decay_rank=m.decay_rank,
                                         eps=cfg.eps), prefix=p + "mix.")
        ff = None if layer.ff is None else PartSpec(
            "swiglu", dict(hidden_size=W, intermediate_size=layer.ff, names=("gate", "up", "down")), prefix=p + "mlp.")
        layers.append(PartSpec("postnorm", dict(mixer=mixer, mixer_norm=norm("norm1", p), alpha=cfg.alpha, feed_forward=ff,
                                                ff_norm=norm("norm2", p, optional=ff is None))))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab, hidden_size=W, tensor="embed", norm=norm("embed.norm"))),
        layers=layers, final_norm=norm("norm", "final."),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=W, tensor="head")),
        eos_token_id=cfg.eos_token_id)


register_architecture(ARCHITECTURE, PofazenConfig.from_dict, pofazen_spec, sizes_from_tensors=True)
