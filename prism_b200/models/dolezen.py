"""Dolezen: a small decoder whose ``config.json`` lists its layers one by one.
Its typed configuration, its layer plan and its entry in the architecture
registry; everything this engine knows about the design by name is here.

The design, as this file builds it from the parts:

* embedding rows times ``embedding.scale``;
* every layer is a *parallel* block: one RMS norm (``l<i>.norm1``), and the
  mixer and the feed-forward both read its output; their results are added
  to the residual stream together;
* mixer ``attention``: grouped-query attention with biases on q, k, v and o,
  no position encoding, an explicit score scale, values of a size of their
  own, a chunked mask (a query sees the earlier keys of its own block of
  ``mask.size`` positions) and a learned sink per head in the softmax's
  denominator; with ``kv_from: j`` the layer has no key and value projections
  and attends over layer j's cache plane with its own queries and mask;
* mixer ``latent_attention``: queries and keys/values through low-rank
  latents, a rotated key part shared by all heads, a sliding window; the cache
  holds the latent and the rotated part only;
* feed-forward ``dense``: up projection, squared relu, down projection;
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
from .decoder import ModelSpec, ScheduleEntry

ARCHITECTURE = "Dolezen"
DEFAULT_MAX_POSITIONS = 131072


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no '{key}'")
    return d[key]


def _pos_int(d: dict, key: str, where: str) -> int:
    v = int(_need(d, key, where))
    if v < 1:
        raise ConfigError(f"config.json: {where}.{key} must be positive, got {v}")
    return v


def _mask_size(mixer: dict, where: str) -> Optional[int]:
    mask = mixer.get("mask")
    if mask is None:
        return None
    return _pos_int(mask, "size", where + ".mask")


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: Optional[int]          # block of positions a query sees (None: every earlier key)
    kv_from: Optional[int]            # layer whose keys and values this layer uses (None: its own)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                          # unrotated query/key size per head
    rot_dim: int                      # rotated part per head
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int                     # entries of the rotated part that turn
    mask_size: Optional[int]          # sliding window (None: every earlier key)


@dataclass(frozen=True)
class DolezenLayer:
    type: str                         # "attention" | "latent_attention"
    mixer: object
    ff: Optional[int]                 # hidden size of the dense feed-forward (None: the layer has none)


@dataclass(frozen=True)
class DolezenConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[DolezenLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "DolezenConfig":
        vocab, width = _pos_int(raw, "vocab", "the model"), _pos_int(raw, "width", "the model")
        eps = float(_need(_need(raw, "norm", "the model"), "eps", "norm"))
        emb = raw.get("embedding") or {}
        layers_raw = _need(raw, "layers", "the model")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            kind, mx = _need(lr, "type", where), _need(lr, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                heads = _pos_int(mx, "heads", mw)
                kvh = int(mx.get("kv_heads") or heads)
                if kvh < 1 or heads % kvh:
                    raise ConfigError(f"config.json: {mw}: heads ({heads}) not divisible by kv_heads ({kvh})")
                dim = _pos_int(mx, "dim", mw)
                src = mx.get("kv_from")
                if src is not None:
                    src = int(src)
                    if not 0 <= src < i or layers[src].type != "attention" or layers[src].mixer.kv_from is not None:
                        raise ConfigError(f"config.json: {mw}.kv_from = {src}: must name an earlier attention layer "
                                          f"with key and value projections of its own")
                    o = layers[src].mixer
                    if (o.kv_heads, o.dim, o.vdim) != (kvh, dim, int(mx.get("vdim") or dim)):
                        raise ConfigError(f"config.json: {mw}: kv_heads, dim and vdim must equal those of layer {src}, "
                                          f"whose keys and values it uses")
                mixer = ChunkedAttentionConfig(heads, kvh, dim, int(mx.get("vdim") or dim), float(_need(mx, "scale", mw)),
                                               _mask_size(mx, mw), src)
            elif kind == "latent_attention":
                rot = mx.get("rot") or {}
                rot_dim = int(mx.get("rot_dim") or 0)
                dims = int(rot.get("dims", rot_dim))
                if dims % 2 or not 0 <= dims <= rot_dim:
                    raise ConfigError(f"config.json: {mw}.rot.dims = {dims}: must be even and at most rot_dim ({rot_dim})")
                mixer = LatentAttentionConfig(
                    _pos_int(mx, "heads", mw), _pos_int(mx, "dim", mw), rot_dim, _pos_int(mx, "vdim", mw),
                    _pos_int(mx, "q_rank", mw), _pos_int(mx, "kv_rank", mw), float(_need(mx, "scale", mw)),
                    float(rot.get("base", 10000.0)), dims, _mask_size(mx, mw))
            else:
                raise ConfigError(f"config.json: {where}.type = {kind!r}: this design has 'attention' and "
                                  f"'latent_attention' mixers")
            mlp = lr.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind = {mlp.get('kind')!r}: only 'dense' is computed")
                ff = _pos_int(mlp, "ff", where + ".mlp")
            layers.append(DolezenLayer(kind, mixer, ff))
        eos = raw.get("eos_token_id")
        eos = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        return cls(vocab, width, eps, float(emb.get("scale", 1.0)), tuple(layers),
                   int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS), eos)


def dolezen_spec(cfg: DolezenConfig) -> ModelSpec:
    W = cfg.width
    # A cache plane gives back the pages of earlier blocks only if every layer that reads it has the same mask.
    family = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            family.setdefault(owner, set()).add(layer.mixer.mask_size)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "attention":
            owner = i if m.kv_from is None else m.kv_from
            sizes = family[owner]
            mixer = PartSpec("gqa_attention", dict(
                hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                qkv_bias=True, o_bias=True, scale=m.scale, chunk=m.mask_size, sink=True, own_kv=m.kv_from is None,
                cache_chunk=next(iter(sizes)) if len(sizes) == 1 else None,
                names=dict(q="q", k="k", v="v", o="o", q_b="q.b", k_b="k.b", v_b="v.b", o_b="o.b", sink="sink")),
                prefix=p + "mix.")
            schedule.append(ScheduleEntry(i, reads_cache_of=m.kv_from))
        else:
            mixer = PartSpec("latent_attention", dict(
                hidden_size=W, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_head_dim=m.vdim,
                q_rank=m.q_rank, kv_rank=m.kv_rank, eps=cfg.eps, rope_base=m.rot_base, rope_dims=m.rot_dims,
                window=m.mask_size, scale=m.scale,
                names=dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o")),
                prefix=p + "mix.")
            schedule.append(ScheduleEntry(i))
        ff = None if layer.ff is None else PartSpec(
            "mlp", dict(hidden_size=W, intermediate_size=layer.ff, activation="relu2", names=("up", "down")),
            prefix=p + "mlp.")
        layers.append(PartSpec("parallel", dict(
            mixer=mixer, feed_forward=ff,
            norm=PartSpec("rmsnorm", dict(width=W, eps=cfg.eps, tensor="norm1"), prefix=p))))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token", dict(vocab_size=cfg.vocab, hidden_size=W, scale=cfg.embedding_scale, tensor="embed")),
        layers=layers, schedule=schedule,
        final_norm=PartSpec("rmsnorm", dict(width=W, eps=cfg.eps, tensor="norm"), prefix="final."),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=W, tensor="head")),
        eos_token_id=cfg.eos_token_id)


register_architecture(ARCHITECTURE, DolezenConfig.from_dict, dolezen_spec)
