"""Typed view of a Bumolix ``config.json``.

Bumolix is a decoder-only model with a nested configuration: ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` and a
list ``layers`` whose entries give the layer's ``type`` (``parallel``: an attention mixer and a gated-linear-attention
mixer side by side, under ``mixer.left`` and ``mixer.right`` with ``left_scale`` and ``right_scale``; ``mamba1``: a
selective-scan mixer), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``: ``kind`` ``dense``, or
null for none).  Every size and constant is read from there; a layer type or feed-forward kind that is not understood
is refused by name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .dosovik_config import _get
from .model_config import ConfigError


@dataclass(frozen=True)
class ChunkAttentionSizes:
    heads: int
    kv_heads: int
    dim: int                     # size of a query / key head
    vdim: int                    # size of a value head
    scale: float
    chunk: Optional[int]         # mask.size: positions see only their own chunk (None: every earlier position)
    rot_dims: int                # how many leading dims of a head rotate (0: no rotation)
    rot_base: float
    rot_factor: float            # rot.scaling.factor: every frequency is divided by it (1: unscaled)


@dataclass(frozen=True)
class LinearAttentionSizes:
    heads: int
    dim: int                     # key channels of a head (rows of its state)
    vdim: int                    # value channels of a head (columns of its state)
    tau: float                   # the decay is sigmoid(z)^(1 / tau)


@dataclass(frozen=True)
class SideBySideSizes:
    left: ChunkAttentionSizes
    right: LinearAttentionSizes
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class Mamba1Sizes:
    inner: int                   # channels of the recurrence
    state: int                   # states per channel
    dt_rank: int                 # width of the low-rank step-size projection
    conv: int                    # taps of the causal convolution


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class BumolixLayer:
    type: str
    mixer: Union[SideBySideSizes, Mamba1Sizes]
    mlp: Optional[DenseFF]


def _positive(v, where: str):
    if v <= 0:
        raise ConfigError(f"config.json {where} must be positive, got {v}")
    return v


def _attention(m: dict, where: str) -> ChunkAttentionSizes:
    pos = lambda key: _positive(_get(m, key, int, where), where + key)  # noqa: E731
    heads, kv_heads, dim = pos("heads"), pos("kv_heads"), pos("dim")
    if heads % kv_heads:
        raise ConfigError(f"config.json {where}heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
    mask = _get(m, "mask", dict, where, required=False)
    chunk = _positive(_get(mask, "size", int, where + "mask."), where + "mask.size") if mask is not None else None
    rot = _get(m, "rot", dict, where, required=False)
    rot_dims = _get(rot, "dims", int, where + "rot.") if rot is not None else 0
    if rot_dims < 0 or rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"config.json {where}rot.dims ({rot_dims}) must be even and at most dim ({dim})")
    scaling = _get(rot, "scaling", dict, where + "rot.", required=False) if rot is not None else None
    factor = _positive(_get(scaling, "factor", float, where + "rot.scaling."), where + "rot.scaling.factor") if scaling is not None else 1.0
    return ChunkAttentionSizes(heads=heads, kv_heads=kv_heads, dim=dim, vdim=pos("vdim"), scale=_get(m, "scale", float, where),
                               chunk=chunk, rot_dims=rot_dims, rot_base=_get(rot, "base", float, where + "rot.") if rot_dims else 1.0,
                               rot_factor=factor)


def _linear_attention(m: dict, where: str) -> LinearAttentionSizes:
    pos = lambda key: _positive(_get(m, key, int, where), where + key)  # noqa: E731
    return LinearAttentionSizes(heads=pos("heads"), dim=pos("dim"), vdim=pos("vdim"),
                                tau=_positive(_get(m, "tau", float, where), where + "tau"))


@dataclass(frozen=True)
class BumolixConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: Tuple[BumolixLayer, ...]

    architecture = "Bumolix"

    @staticmethod
    def from_dict(d: dict) -> "BumolixConfig":
        if not isinstance(d.get("layers"), list) or not d["layers"]:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers = []
        for i, ly in enumerate(d["layers"]):
            where = f"layers[{i}]."
            kind = _get(ly, "type", str, where)
            m = _get(ly, "mixer", dict, where)
            mw = where + "mixer."
            if kind == "parallel":
                mixer = SideBySideSizes(
                    left=_attention(_get(m, "left", dict, mw), mw + "left."),
                    right=_linear_attention(_get(m, "right", dict, mw), mw + "right."),
                    left_scale=_get(m, "left_scale", float, mw, default=1.0, required=False),
                    right_scale=_get(m, "right_scale", float, mw, default=1.0, required=False))
            elif kind == "mamba1":
                pos = lambda key: _positive(_get(m, key, int, mw), mw + key)  # noqa: E731
                mixer = Mamba1Sizes(inner=pos("inner"), state=pos("state"), dt_rank=pos("dt_rank"), conv=pos("conv"))
            else:
                raise ConfigError(f"config.json {where}type {kind!r} is not a mixer of this design "
                                  f"(known: 'parallel', 'mamba1')")
            mlp = ly.get("mlp")
            if mlp is not None:
                ff_kind = _get(mlp, "kind", str, where + "mlp.")
                if ff_kind != "dense":
                    raise ConfigError(f"config.json {where}mlp.kind {ff_kind!r} is not known (known: 'dense')")
                mlp = DenseFF(ff=_positive(_get(mlp, "ff", int, where + "mlp."), where + "mlp.ff"))
            layers.append(BumolixLayer(kind, mixer, mlp))
        return BumolixConfig(
            vocab=_positive(_get(d, "vocab", int, ""), "vocab"), width=_positive(_get(d, "width", int, ""), "width"),
            eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
            residual_mult=_get(d, "residual_mult", float, "", default=1.0, required=False), layers=tuple(layers))
