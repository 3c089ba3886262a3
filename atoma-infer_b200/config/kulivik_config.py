"""Typed view of a Kulivik ``config.json``.

Kulivik is a decoder-only model with a nested configuration: ``vocab``, ``width``, ``norm.eps``, ``logit_scale``,
``logit_softcap`` and a list ``layers`` whose entries give the layer's ``type`` (``attention_2``: rotated, windowed
attention; ``attention``: attention behind a short convolution, with a sink; ``parallel``: an attention mixer and a
linear-attention mixer with constant decays side by side, under ``mixer.left`` and ``mixer.right``), the mixer's sizes and
constants (``mixer``) and its feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for none).  Every size and
constant is read from there; what a layer's entry does not mention is off; a layer type or feed-forward kind that is not
understood is refused by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .dosovik_config import _get
from .model_config import ConfigError


@dataclass(frozen=True)
class HeadSizes:
    heads: int
    kv_heads: int
    dim: int                     # size of a query / key head
    vdim: int                    # size of a value head
    scale: float


@dataclass(frozen=True)
class RotaryWindowAttention:     # type "attention_2"
    sizes: HeadSizes
    softcap: Optional[float]     # score <- softcap * tanh(score / softcap)
    window: Optional[int]        # mask.size
    keep_first: int              # mask.keep_first
    rot_dims: int                # 0: no rotation
    rot_base: float
    v_mix: bool


@dataclass(frozen=True)
class ConvSinkAttention:         # type "attention"
    sizes: HeadSizes
    conv: int                    # taps of the convolution on q, k, v (0 or 1: none)
    v_mix: bool


@dataclass(frozen=True)
class BiasedAttention:           # the left side of type "parallel"
    sizes: HeadSizes
    q_temp: Optional[Tuple[float, int]]   # (coef, every)


@dataclass(frozen=True)
class DecaySizes:                # the right side of type "parallel"
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class SideBySideSizes:
    left: BiasedAttention
    right: DecaySizes
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseFF:
    ff: int
    limit: float


@dataclass(frozen=True)
class ExpertsFF:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class KulivikLayer:
    type: str
    mixer: Union[RotaryWindowAttention, ConvSinkAttention, SideBySideSizes]
    mlp: Union[None, DenseFF, ExpertsFF]


def _positive(v, where: str):
    if v <= 0:
        raise ConfigError(f"config.json {where} must be positive, got {v}")
    return v


def _heads(m: dict, where: str) -> HeadSizes:
    pos = lambda key: _positive(_get(m, key, int, where), where + key)  # noqa: E731
    heads, kv_heads = pos("heads"), pos("kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"config.json {where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    return HeadSizes(heads=heads, kv_heads=kv_heads, dim=pos("dim"), vdim=pos("vdim"), scale=_get(m, "scale", float, where))


def _rotary_window(m: dict, where: str) -> RotaryWindowAttention:
    sizes = _heads(m, where)
    mask = _get(m, "mask", dict, where, required=False)
    window = _positive(_get(mask, "size", int, where + "mask."), where + "mask.size") if mask is not None else None
    keep = _get(mask, "keep_first", int, where + "mask.", default=0, required=False) if mask is not None else 0
    if keep < 0:
        raise ConfigError(f"config.json {where}mask.keep_first must not be negative, got {keep}")
    rot = _get(m, "rot", dict, where, required=False)
    rot_dims = _get(rot, "dims", int, where + "rot.") if rot is not None else 0
    if rot_dims < 0 or rot_dims % 2 or rot_dims > sizes.dim:
        raise ConfigError(f"config.json {where}rot.dims ({rot_dims}) must be even and at most dim ({sizes.dim})")
    cap = _get(m, "softcap", float, where, required=False)
    return RotaryWindowAttention(sizes=sizes, softcap=_positive(cap, where + "softcap") if cap is not None else None,
                                 window=window, keep_first=keep, rot_dims=rot_dims,
                                 rot_base=_positive(_get(rot, "base", float, where + "rot."), where + "rot.base") if rot_dims else 1.0,
                                 v_mix=bool(m.get("v_mix", False)))


def _side_by_side(m: dict, where: str) -> SideBySideSizes:
    lw, rw = where + "left.", where + "right."
    left, right = _get(m, "left", dict, where), _get(m, "right", dict, where)
    qt = _get(left, "q_temp", dict, lw, required=False)
    q_temp = ((_get(qt, "coef", float, lw + "q_temp."), _positive(_get(qt, "every", int, lw + "q_temp."), lw + "q_temp.every"))
              if qt is not None else None)
    pos = lambda key: _positive(_get(right, key, int, rw), rw + key)  # noqa: E731
    heads = pos("heads")
    decay = right.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(a, (int, float)) and not isinstance(a, bool) for a in decay):
        raise ConfigError(f"config.json {rw}decay must list one number per head ({heads})")
    return SideBySideSizes(left=BiasedAttention(_heads(left, lw), q_temp),
                           right=DecaySizes(heads=heads, dim=pos("dim"), vdim=pos("vdim"), decay=tuple(float(a) for a in decay)),
                           left_scale=_get(m, "left_scale", float, where, default=1.0, required=False),
                           right_scale=_get(m, "right_scale", float, where, default=1.0, required=False))


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    kind = _get(mlp, "kind", str, where)
    if kind == "dense":
        return DenseFF(ff=_positive(_get(mlp, "ff", int, where), where + "ff"),
                       limit=_positive(_get(mlp, "limit", float, where), where + "limit"))
    if kind == "moe":
        e, r = _get(mlp, "expert", dict, where), _get(mlp, "router", dict, where)
        experts = _positive(_get(r, "experts", int, where + "router."), where + "router.experts")
        top = _positive(_get(r, "top", int, where + "router."), where + "router.top")
        if top > experts:
            raise ConfigError(f"config.json {where}router.top ({top}) must not exceed router.experts ({experts})")
        return ExpertsFF(ff=_positive(_get(e, "ff", int, where + "expert."), where + "expert.ff"), experts=experts, top=top)
    raise ConfigError(f"config.json {where}kind {kind!r} is not known (known: 'dense', 'moe')")


@dataclass(frozen=True)
class KulivikConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    logit_softcap: Optional[float]
    layers: Tuple[KulivikLayer, ...]

    architecture = "Kulivik"

    @staticmethod
    def from_dict(d: dict) -> "KulivikConfig":
        if not isinstance(d.get("layers"), list) or not d["layers"]:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers = []
        for i, ly in enumerate(d["layers"]):
            where = f"layers[{i}]."
            kind = _get(ly, "type", str, where)
            m, mw = _get(ly, "mixer", dict, where), where + "mixer."
            if kind == "attention_2":
                mixer = _rotary_window(m, mw)
            elif kind == "attention":
                conv = _get(m, "conv", int, mw, default=0, required=False)
                if conv < 0:
                    raise ConfigError(f"config.json {mw}conv must not be negative, got {conv}")
                mixer = ConvSinkAttention(sizes=_heads(m, mw), conv=conv, v_mix=bool(m.get("v_mix", False)))
            elif kind == "parallel":
                mixer = _side_by_side(m, mw)
            else:
                raise ConfigError(f"config.json {where}type {kind!r} is not a mixer of this design "
                                  f"(known: 'attention', 'attention_2', 'parallel')")
            layers.append(KulivikLayer(kind, mixer, _mlp(ly.get("mlp"), where + "mlp.")))
        cap = _get(d, "logit_softcap", float, "", required=False)
        return KulivikConfig(
            vocab=_positive(_get(d, "vocab", int, ""), "vocab"), width=_positive(_get(d, "width", int, ""), "width"),
            eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
            logit_scale=_get(d, "logit_scale", float, "", default=1.0, required=False),
            logit_softcap=_positive(cap, "logit_softcap") if cap is not None else None, layers=tuple(layers))
