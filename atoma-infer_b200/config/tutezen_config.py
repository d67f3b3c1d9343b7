"""Typed view of a Tutezen ``config.json``.

Tutezen is a decoder-only model with a nested configuration: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``,
an optional ``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1 run that many times in a row) and a list
``layers`` whose entries give the layer's ``type`` (``mamba2`` or ``latent_attention``), the mixer's sizes and
constants (``mixer``) and its feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for none).  Every size and
constant is read from there; a key that would change the math and is not understood is refused.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple, Union

from .dosovik_config import _get
from .model_config import ConfigError


@dataclass(frozen=True)
class Mamba2Sizes:
    heads: int
    vdim: int          # size of a head
    state: int         # N: rows of a head's state matrix
    groups: int        # heads of one group share B and C
    conv: int          # taps of the causal convolution
    norm_groups: int   # the gated output is normalised in this many equal parts


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int                  # unrotated query/key dimensions of a head
    rot_dim: int              # rotated query/key dimensions of a head (the key part is shared by all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]     # mask.size: a position sees itself and the window - 1 before it (None: all)
    rot_dims: int             # how many leading dimensions of the rotated part turn (0: none)
    rot_base: float


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class MoEFF:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int            # 0: no shared expert


@dataclass(frozen=True)
class TutezenLayer:
    type: str
    mixer: Union[Mamba2Sizes, LatentAttentionSizes]
    mlp: Union[DenseFF, MoEFF, None]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TutezenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    loop: Optional[Loop]
    layers: Tuple[TutezenLayer, ...]

    architecture = "Tutezen"

    @staticmethod
    def from_dict(d: dict) -> "TutezenConfig":
        if not isinstance(d.get("layers"), list) or not d["layers"]:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        layers = []
        for i, ly in enumerate(d["layers"]):
            where = f"layers[{i}]."
            kind = _get(ly, "type", str, where)
            m = _get(ly, "mixer", dict, where)
            mw = where + "mixer."
            pos = lambda key: _positive(_get(m, key, int, mw), mw + key)  # noqa: E731
            if kind == "mamba2":
                mixer = Mamba2Sizes(heads=pos("heads"), vdim=pos("vdim"), state=pos("state"), groups=pos("groups"),
                                    conv=pos("conv"), norm_groups=pos("norm_groups"))
                if mixer.heads % mixer.groups:
                    raise ConfigError(f"config.json {mw}heads ({mixer.heads}) must be a multiple of groups ({mixer.groups})")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json {mw}norm_groups ({mixer.norm_groups}) must divide heads * vdim")
            elif kind == "latent_attention":
                mask = _get(m, "mask", dict, mw, required=False)
                window = _positive(_get(mask, "size", int, mw + "mask."), mw + "mask.size") if mask is not None else None
                rot = _get(m, "rot", dict, mw, required=False)
                rot_dim = pos("rot_dim")
                rot_dims = _get(rot, "dims", int, mw + "rot.") if rot is not None else 0
                if rot_dims < 0 or rot_dims % 2 or rot_dims > rot_dim:
                    raise ConfigError(f"config.json {mw}rot.dims ({rot_dims}) must be even and at most rot_dim ({rot_dim})")
                mixer = LatentAttentionSizes(
                    heads=pos("heads"), dim=pos("dim"), rot_dim=rot_dim, vdim=pos("vdim"), q_rank=pos("q_rank"),
                    kv_rank=pos("kv_rank"), scale=_get(m, "scale", float, mw), window=window, rot_dims=rot_dims,
                    rot_base=_get(rot, "base", float, mw + "rot.") if rot is not None else 1.0)
            else:
                raise ConfigError(f"config.json {where}type {kind!r} is not a mixer of this design "
                                  f"(known: 'mamba2', 'latent_attention')")
            layers.append(TutezenLayer(kind, mixer, _feed_forward(ly.get("mlp"), where + "mlp.")))
        loop = _get(d, "loop", dict, "", required=False)
        if loop is not None:
            loop = Loop(_get(loop, "start", int, "loop."), _get(loop, "stop", int, "loop."), _get(loop, "times", int, "loop."))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError(f"config.json loop {loop} does not fit {len(layers)} layers")
        return TutezenConfig(
            vocab=_positive(_get(d, "vocab", int, ""), "vocab"), width=_positive(_get(d, "width", int, ""), "width"),
            eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
            residual_mult=_get(d, "residual_mult", float, "", default=1.0, required=False), loop=loop, layers=tuple(layers))


def _positive(v: int, where: str) -> int:
    if v <= 0:
        raise ConfigError(f"config.json {where} must be positive, got {v}")
    return v


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = _get(mlp, "kind", str, where)
    if kind == "dense":
        return DenseFF(ff=_positive(_get(mlp, "ff", int, where), where + "ff"))
    if kind == "moe":
        router = _get(mlp, "router", dict, where)
        experts = _positive(_get(router, "experts", int, where + "router."), where + "router.experts")
        top = _positive(_get(router, "top", int, where + "router."), where + "router.top")
        if top > experts:
            raise ConfigError(f"config.json {where}router.top ({top}) exceeds router.experts ({experts})")
        shared = _get(mlp, "shared", dict, where, required=False)
        return MoEFF(experts=experts, top=top,
                     expert_ff=_positive(_get(_get(mlp, "expert", dict, where), "ff", int, where + "expert."), where + "expert.ff"),
                     shared_ff=_positive(_get(shared, "ff", int, where + "shared."), where + "shared.ff") if shared is not None else 0)
    raise ConfigError(f"config.json {where}kind {kind!r} is not known (known: 'dense', 'moe')")
