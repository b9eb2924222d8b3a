"""Typed configuration of the Burinex design, read from its own config.json keys.

A Burinex model is a list of layers between a token embedding and a final RMS norm with a head of its own, whose
logits are capped by a tanh. A layer puts its norm AFTER the residual sum: x = norm1(alpha x + s1 (.) mixer(x)), then,
where it has a feed-forward, x = norm2(alpha x + s2 (.) ff(x)), with one constant alpha for the whole model and learned
scales s per channel. Three kinds of mixer: "attention" (grouped queries without rotation, RMS norms over the whole query
and key projections, a temperature on the queries that grows with the position, a softmax with one more term exp(0),
one sigmoid gate per head), "latent_attention" (queries through a normed latent of their own; keys and values from a
cached normed latent plus one rotated key part shared by all heads, YaRN-scaled rotation, a sliding window, a learned
term per head in the softmax's denominator) and "lightning" (linear attention with a constant decay per head over a
matrix state, one norm over the concatenated heads, a sigmoid gate per channel). The feed-forward is a mixture of
experts under a sigmoid router whose weights multiply what the experts read, with a shared expert. Every layer carries
its own sizes and constants; nothing has a default in code: a missing or ill-typed key is a `ConfigError` that names it.

    architecture      "Burinex"
    vocab, width, postln_alpha, logit_softcap (null or absent: no cap)
    norm.eps          the epsilon of every RMS norm of the model
    layers[i].type    "attention" | "latent_attention" | "lightning"
    layers[i].mixer   attention: heads, kv_heads, dim, vdim, scale, q_temp {coef, every} or null
                      latent_attention: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask {size} or null,
                                        rot {base, dims, scaling {factor, original, fast, slow} or null}
                      lightning: heads, dim, vdim, decay [one constant per head]
    layers[i].mlp     null | {kind: "moe", router {experts, top}, expert {ff}, shared {ff} or null}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .registry import ConfigError
from .zemivik import _num, _obj, _pos_int


@dataclass(frozen=True)
class GatedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: Optional[float]      # None = no temperature on the queries
    temp_every: Optional[int]


@dataclass(frozen=True)
class YarnScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: Optional[int]           # None = queries straight from the layer's input
    scale: float
    window: int                     # 0 = every earlier token
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[YarnScaling]


@dataclass(frozen=True)
class Lightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    expert_ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class BurinexLayer:
    type: str
    mixer: Union[GatedAttention, LatentAttention, Lightning]
    mlp: Optional[RoutedFF]


MIXER_TYPES = ("attention", "latent_attention", "lightning")


def _attention(d: dict, where: str) -> GatedAttention:
    heads, kv_heads = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    coef = every = None
    if d.get("q_temp") is not None:
        t = _obj(d["q_temp"], where + "'q_temp'")
        coef, every = _num(t, "coef", where + "q_temp.", float), _pos_int(t, "every", where + "q_temp.")
    return GatedAttention(heads=heads, kv_heads=kv_heads, dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                          scale=_num(d, "scale", where, float), temp_coef=coef, temp_every=every)


def _latent_attention(d: dict, where: str) -> LatentAttention:
    rot = _obj(d.get("rot"), where + "'rot'")
    rot_dim, rot_dims = _pos_int(d, "rot_dim", where), _pos_int(rot, "dims", where + "rot.")
    if rot_dims % 2 or rot_dims > rot_dim:
        raise ConfigError(f"config.json: key {where}rot.'dims' ({rot_dims}) must be even and at most 'rot_dim' ({rot_dim})")
    base = _num(rot, "base", where + "rot.", float)
    if base <= 1:
        raise ConfigError(f"config.json: key {where}rot.'base' must exceed 1, got {base}")
    scaling = None
    if rot.get("scaling") is not None:
        s = _obj(rot["scaling"], where + "rot.'scaling'")
        w = where + "rot.scaling."
        scaling = YarnScaling(factor=_num(s, "factor", w, float), original=_num(s, "original", w, float),
                              fast=_num(s, "fast", w, float), slow=_num(s, "slow", w, float))
        for key in ("factor", "original", "fast", "slow"):
            if getattr(scaling, key) <= 0:
                raise ConfigError(f"config.json: key {w}{key!r} must be positive, got {getattr(scaling, key)}")
    window = 0
    if d.get("mask") is not None:
        window = _pos_int(_obj(d["mask"], where + "'mask'"), "size", where + "mask.")
    q_rank = _pos_int(d, "q_rank", where) if d.get("q_rank") is not None else None
    return LatentAttention(heads=_pos_int(d, "heads", where), dim=_pos_int(d, "dim", where), rot_dim=rot_dim,
                           vdim=_pos_int(d, "vdim", where), kv_rank=_pos_int(d, "kv_rank", where), q_rank=q_rank,
                           scale=_num(d, "scale", where, float), window=window, rot_base=base, rot_dims=rot_dims,
                           rot_scaling=scaling)


def _lightning(d: dict, where: str) -> Lightning:
    heads = _pos_int(d, "heads", where)
    decay = d.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or \
            not all(isinstance(a, (int, float)) and not isinstance(a, bool) for a in decay):
        raise ConfigError(f"config.json: key {where}'decay' must be a list of {heads} numbers (one per head), got {decay!r}")
    return Lightning(heads=heads, dim=_pos_int(d, "dim", where), vdim=_pos_int(d, "vdim", where),
                     decay=tuple(float(a) for a in decay))


def _mlp(m, where: str) -> Optional[RoutedFF]:
    if m is None:
        return None
    m = _obj(m, where + "'mlp'")
    if m.get("kind") != "moe":
        raise ConfigError(f"config.json: key {where}mlp.'kind' must be 'moe', got {m.get('kind')!r}")
    router = _obj(m.get("router"), where + "mlp.'router'")
    experts, top = _pos_int(router, "experts", where + "mlp.router."), _pos_int(router, "top", where + "mlp.router.")
    if top > experts:
        raise ConfigError(f"config.json: key {where}mlp.router.'top' ({top}) exceeds 'experts' ({experts})")
    shared = m.get("shared")
    shared_ff = None if shared is None else _pos_int(_obj(shared, where + "mlp.'shared'"), "ff", where + "mlp.shared.")
    return RoutedFF(experts=experts, top=top,
                    expert_ff=_pos_int(_obj(m.get("expert"), where + "mlp.'expert'"), "ff", where + "mlp.expert."),
                    shared_ff=shared_ff)


@dataclass(frozen=True)
class BurinexConfig:
    vocab: int
    width: int
    alpha: float
    logit_softcap: Optional[float]
    norm_eps: float
    layers: Tuple[BurinexLayer, ...]

    @staticmethod
    def from_dict(cfg: dict) -> "BurinexConfig":
        layers_json = cfg.get("layers")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        readers = {"attention": _attention, "latent_attention": _latent_attention, "lightning": _lightning}
        layers = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            e = _obj(entry, f"layers[{i}]")
            kind = e.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: key {where}'type' must be one of {list(MIXER_TYPES)}, got {kind!r}")
            mixer = readers[kind](_obj(e.get("mixer"), where + "'mixer'"), where + "mixer.")
            layers.append(BurinexLayer(type=kind, mixer=mixer, mlp=_mlp(e.get("mlp"), where)))
        cap = None
        if cfg.get("logit_softcap") is not None:
            cap = _num(cfg, "logit_softcap", "", float)
            if cap <= 0:
                raise ConfigError(f"config.json: key 'logit_softcap' must be positive, got {cap}")
        return BurinexConfig(vocab=_pos_int(cfg, "vocab", ""), width=_pos_int(cfg, "width", ""),
                             alpha=_num(cfg, "postln_alpha", "", float), logit_softcap=cap,
                             norm_eps=_num(_obj(cfg.get("norm"), "'norm'"), "eps", "norm.", float), layers=tuple(layers))
