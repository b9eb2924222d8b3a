"""Typed configuration of the Ganupel design, read from its own config.json keys.

A Ganupel model is a list of layers between a token embedding and a final norm with a head of its own. A layer is
x += s1 (.) mixer(norm(x)), then x += s2 (.) ff(norm(x)) where it has a feed-forward, with s1 and s2 learned scales
per channel and norms whose weights are stored around zero. Two kinds of layer: "parallel" (two mixers side by side,
an attention with rotated queries and keys whose weights are sigmoids instead of a softmax, and a gated linear
recurrence over a matrix state; their outputs are added with a constant each) and "rglru" (a real-gated linear
recurrent unit behind a short causal convolution). Two feed-forwards: a dense one whose activation is a sum of
normalised powers, and routed experts (square of relu) some of whose router outputs stand for experts that return
their input. Every layer carries its own sizes and constants; nothing has a default in code: a missing or ill-typed
key is a `ConfigError` that names it.

    architecture      "Ganupel"
    vocab, width
    norm.eps          the epsilon of every RMS norm of the model
    layers[i].type    "parallel" | "rglru"
    layers[i].mixer   parallel: left {heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size} or null},
                                right {heads, dim, vdim}, left_scale, right_scale
                      rglru:    width, blocks, conv
    layers[i].mlp     null | {kind: "dense", ff} | {kind: "moe", router {experts, identity, top, scale}, expert {ff}}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple, Union

from .registry import ConfigError
from .zemivik import _num, _obj, _pos_int


@dataclass(frozen=True)
class SigmoidAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    window: int                     # 0 = every earlier token


@dataclass(frozen=True)
class MatrixRecurrence:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class ParallelMixers:
    left: SigmoidAttention
    right: MatrixRecurrence
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class RecurrentUnit:
    width: int
    blocks: int
    taps: int


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    identity: int
    top: int
    scale: float
    expert_ff: int


@dataclass(frozen=True)
class GanupelLayer:
    type: str
    mixer: Union[ParallelMixers, RecurrentUnit]
    mlp: Union[None, DenseFF, RoutedFF]


MIXER_TYPES = ("parallel", "rglru")
MLP_KINDS = ("dense", "moe")


def _attention(d: dict, where: str) -> SigmoidAttention:
    heads, kv_heads = _pos_int(d, "heads", where), _pos_int(d, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}'heads' ({heads}) must be a multiple of 'kv_heads' ({kv_heads})")
    dim = _pos_int(d, "dim", where)
    rot = _obj(d.get("rot"), where + "'rot'")
    rot_dims = _pos_int(rot, "dims", where + "rot.")
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"config.json: key {where}rot.'dims' ({rot_dims}) must be even and at most 'dim' ({dim})")
    window = 0
    if d.get("mask") is not None:
        window = _pos_int(_obj(d["mask"], where + "'mask'"), "size", where + "mask.")
    return SigmoidAttention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_pos_int(d, "vdim", where),
                            scale=_num(d, "scale", where, float), rot_base=_num(rot, "base", where + "rot.", float),
                            rot_dims=rot_dims, window=window)


def _mixer(kind: str, m: dict, where: str):
    if kind == "parallel":
        right = _obj(m.get("right"), where + "'right'")
        return ParallelMixers(
            left=_attention(_obj(m.get("left"), where + "'left'"), where + "left."),
            right=MatrixRecurrence(heads=_pos_int(right, "heads", where + "right."),
                                   dim=_pos_int(right, "dim", where + "right."),
                                   vdim=_pos_int(right, "vdim", where + "right.")),
            left_scale=_num(m, "left_scale", where, float), right_scale=_num(m, "right_scale", where, float))
    width, blocks = _pos_int(m, "width", where), _pos_int(m, "blocks", where)
    if width % blocks:
        raise ConfigError(f"config.json: {where}'width' ({width}) must be a multiple of 'blocks' ({blocks})")
    return RecurrentUnit(width=width, blocks=blocks, taps=_pos_int(m, "conv", where))


def _mlp(m, where: str):
    if m is None:
        return None
    m = _obj(m, where + "'mlp'")
    kind = m.get("kind")
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: key {where}mlp.'kind' must be one of {list(MLP_KINDS)}, got {kind!r}")
    if kind == "dense":
        return DenseFF(ff=_pos_int(m, "ff", where + "mlp."))
    router = _obj(m.get("router"), where + "mlp.'router'")
    experts, top = _pos_int(router, "experts", where + "mlp.router."), _pos_int(router, "top", where + "mlp.router.")
    identity = _num(router, "identity", where + "mlp.router.", int)
    if identity < 0:
        raise ConfigError(f"config.json: key {where}mlp.router.'identity' must not be negative, got {identity}")
    if top > experts + identity:
        raise ConfigError(f"config.json: key {where}mlp.router.'top' ({top}) exceeds the router's "
                          f"{experts + identity} outputs")
    return RoutedFF(experts=experts, identity=identity, top=top, scale=_num(router, "scale", where + "mlp.router.", float),
                    expert_ff=_pos_int(_obj(m.get("expert"), where + "mlp.'expert'"), "ff", where + "mlp.expert."))


@dataclass(frozen=True)
class GanupelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[GanupelLayer, ...]

    @staticmethod
    def from_dict(cfg: dict) -> "GanupelConfig":
        layers_json = cfg.get("layers")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            e = _obj(entry, f"layers[{i}]")
            kind = e.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: key {where}'type' must be one of {list(MIXER_TYPES)}, got {kind!r}")
            mixer = _mixer(kind, _obj(e.get("mixer"), where + "'mixer'"), where + "mixer.")
            layers.append(GanupelLayer(type=kind, mixer=mixer, mlp=_mlp(e.get("mlp"), where)))
        return GanupelConfig(vocab=_pos_int(cfg, "vocab", ""), width=_pos_int(cfg, "width", ""),
                             norm_eps=_num(_obj(cfg.get("norm"), "'norm'"), "eps", "norm.", float), layers=tuple(layers))
