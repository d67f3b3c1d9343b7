"""Typed view of a Dosovik ``config.json``.

Dosovik is a decoder-only model whose configuration is nested: ``vocab``, ``width``, ``norm.eps``,
``postln_alpha``, ``embedding.scale``, ``canon.taps`` and a list ``layers`` whose entries give the layer's ``type``
(which mixer it has), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``, or null for none).
Every size and constant is read from there; a key that would change the math and is not understood is refused.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError


def _get(d: dict, key: str, typ, where: str, default=None, required: bool = True):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json is missing {where}{key!r}")
        return default
    v = d[key]
    if typ is int and (isinstance(v, bool) or not isinstance(v, int)):
        raise ConfigError(f"config.json key {where}{key!r} must be an integer, got {v!r}")
    if typ is float and (isinstance(v, bool) or not isinstance(v, (int, float))):
        raise ConfigError(f"config.json key {where}{key!r} must be a number, got {v!r}")
    if typ is dict and not isinstance(v, dict):
        raise ConfigError(f"config.json key {where}{key!r} must be an object, got {v!r}")
    return typ(v) if typ in (int, float) else v


@dataclass(frozen=True)
class DosovikAttention:
    heads: int
    kv_heads: int
    dim: int                     # size of a query / key head
    vdim: int                    # size of a value head
    scale: float
    chunk: Optional[int]         # mask.size: positions see only their own chunk (None: every earlier position)
    rot_dims: Optional[int]      # how many leading dims of a head rotate (None: no rotation)
    rot_base: float
    v_mix: bool


@dataclass(frozen=True)
class DosovikDense:
    ff: int


@dataclass(frozen=True)
class DosovikLayer:
    type: str
    mixer: DosovikAttention
    mlp: Optional[DosovikDense]


@dataclass(frozen=True)
class DosovikConfig:
    vocab: int
    width: int
    eps: float
    alpha: float
    embedding_scale: float
    taps: Optional[int]          # canon.taps (None: sublayers read the stream itself)
    layers: Tuple[DosovikLayer, ...]

    architecture = "Dosovik"

    @staticmethod
    def from_dict(d: dict) -> "DosovikConfig":
        if not isinstance(d.get("layers"), list) or not d["layers"]:
            raise ConfigError("config.json needs a non-empty list 'layers'")
        width = _get(d, "width", int, "")
        layers = []
        for i, ly in enumerate(d["layers"]):
            where = f"layers[{i}]."
            kind = _get(ly, "type", str, where)
            if kind != "attention":
                raise ConfigError(f"config.json {where}type {kind!r} is not a mixer of this design (known: 'attention')")
            m = _get(ly, "mixer", dict, where)
            mw = where + "mixer."
            heads, kv = _get(m, "heads", int, mw), _get(m, "kv_heads", int, mw)
            if heads <= 0 or kv <= 0 or heads % kv:
                raise ConfigError(f"config.json {mw}heads ({heads}) must be a positive multiple of kv_heads ({kv})")
            mask = _get(m, "mask", dict, mw, required=False)
            chunk = _get(mask, "size", int, mw + "mask.") if mask is not None else None
            if chunk is not None and chunk <= 0:
                raise ConfigError(f"config.json {mw}mask.size must be positive")
            rot = _get(m, "rot", dict, mw, required=False)
            dim = _get(m, "dim", int, mw)
            rot_dims = _get(rot, "dims", int, mw + "rot.") if rot is not None else None
            if rot_dims is not None and (rot_dims <= 0 or rot_dims % 2 or rot_dims > dim):
                raise ConfigError(f"config.json {mw}rot.dims ({rot_dims}) must be even, positive and at most dim ({dim})")
            att = DosovikAttention(
                heads=heads, kv_heads=kv, dim=dim, vdim=_get(m, "vdim", int, mw), scale=_get(m, "scale", float, mw),
                chunk=chunk, rot_dims=rot_dims, rot_base=_get(rot, "base", float, mw + "rot.") if rot is not None else 1.0,
                v_mix=bool(m.get("v_mix", False)))
            mlp = ly.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", str, where + "mlp.")
                if mk != "dense":
                    raise ConfigError(f"config.json {where}mlp.kind {mk!r} is not known (known: 'dense')")
                mlp = DosovikDense(ff=_get(mlp, "ff", int, where + "mlp."))
            layers.append(DosovikLayer(kind, att, mlp))
        canon = _get(d, "canon", dict, "", required=False)
        emb = _get(d, "embedding", dict, "", required=False)
        return DosovikConfig(
            vocab=_get(d, "vocab", int, ""), width=width, eps=_get(_get(d, "norm", dict, ""), "eps", float, "norm."),
            alpha=_get(d, "postln_alpha", float, "", default=1.0, required=False),
            embedding_scale=_get(emb, "scale", float, "embedding.", default=1.0, required=False) if emb is not None else 1.0,
            taps=_get(canon, "taps", int, "canon.") if canon is not None else None, layers=tuple(layers))
