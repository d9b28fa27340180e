"""Typed configuration of Lamisun, read from its config.json keys.

A Lamisun config.json has ``architecture`` ("Lamisun"), ``vocab``, ``width``, ``norm.eps``,
``embedding`` (``scale``, and optionally ``bigram`` with ``buckets``, ``mul_prev``, ``mul_cur``:
a second table indexed by a hash of a token and the one before it), optionally ``canon.taps``
(a causal convolution over time on what every sublayer reads) and a list ``layers``. Every layer
entry gives its ``type`` (the mixer it has), the mixer's sizes under ``mixer`` and its
feed-forward under ``mlp`` (null: none). The mixers of the design: ``latent_attention``
(softmax attention whose keys and values come from one small latent per token, with a rotated
key part that all heads share and a sigmoid gate on the output) and ``attention`` (grouped-query
differential attention: two score maps per head, queries and keys normed per head, no rotation,
optionally within chunks of ``mask.size`` positions).

Nothing here has a default that stands for a size: a key that the design requires and that is
absent is an error with the key's path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .base import ConfigError, divisible, positive, positive_int

NAME = "Lamisun"


def _need(data: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(data, Mapping) or key not in data:
        raise ConfigError(f"{where}{key} is missing")
    return data[key]


def _sizes(data, keys, where):
    out = []
    for key in keys:
        value = _need(data, key, where)
        positive_int(where + key, value)
        out.append(value)
    return out


@dataclass(frozen=True)
class Rotary:
    base: float
    dims: int

    @classmethod
    def from_dict(cls, data, where):
        (dims,) = _sizes(data, ("dims",), where)
        if dims % 2:
            raise ConfigError(f"{where}dims ({dims}) must be even")
        base = float(_need(data, "base", where))
        positive(where + "base", base)
        return cls(base, dims)

    def to_dict(self):
        return {"base": self.base, "dims": self.dims}


@dataclass(frozen=True)
class LatentMixer:
    """``heads`` heads with ``dim`` unrotated and ``rot_dim`` rotated query/key dimensions, values
    of ``vdim``, a latent of ``kv_rank`` per token."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: Rotary

    @classmethod
    def from_dict(cls, data, where):
        heads, dim, rot_dim, vdim, kv_rank = _sizes(
            data, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), where)
        scale = float(_need(data, "scale", where))
        positive(where + "scale", scale)
        rot = Rotary.from_dict(_need(data, "rot", where), where + "rot.")
        if rot.dims > rot_dim:
            raise ConfigError(f"{where}rot.dims ({rot.dims}) exceeds {where}rot_dim ({rot_dim})")
        return cls(heads, dim, rot_dim, vdim, kv_rank, scale, rot)

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank,
                "rot": self.rot.to_dict(), "rot_dim": self.rot_dim, "scale": self.scale,
                "vdim": self.vdim}


@dataclass(frozen=True)
class DifferentialMixer:
    """``heads`` query heads over ``kv_heads`` key/value heads, two maps of ``dim`` each, values
    of ``vdim``; ``diff`` the constant in the maps' mixing factor; ``chunk`` (None: plain causal)
    the size of the chunks within which positions see each other."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: int | None

    @classmethod
    def from_dict(cls, data, where):
        heads, kv_heads, dim, vdim = _sizes(data, ("heads", "kv_heads", "dim", "vdim"), where)
        divisible(where + "heads", heads, where + "kv_heads", kv_heads)
        scale = float(_need(data, "scale", where))
        positive(where + "scale", scale)
        diff = float(_need(data, "diff", where))
        chunk = None
        if data.get("mask") is not None:
            (chunk,) = _sizes(data["mask"], ("size",), where + "mask.")
        return cls(heads, kv_heads, dim, vdim, scale, diff, chunk)

    def to_dict(self):
        out = {"diff": self.diff, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
               "scale": self.scale, "vdim": self.vdim}
        if self.chunk is not None:
            out["mask"] = {"size": self.chunk}
        return out


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


MIXERS = {"latent_attention": LatentMixer, "attention": DifferentialMixer}


@dataclass(frozen=True)
class LamisunLayer:
    type: str
    mixer: Any                      # LatentMixer or DifferentialMixer
    mlp: DenseFeedForward | None

    @classmethod
    def from_dict(cls, data, where):
        kind = _need(data, "type", where)
        if kind not in MIXERS:
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design "
                              f"({', '.join(sorted(MIXERS))})")
        mixer = MIXERS[kind].from_dict(_need(data, "mixer", where), where + "mixer.")
        mlp = data.get("mlp")
        if mlp is not None:
            form = _need(mlp, "kind", where + "mlp.")
            if form != "dense":
                raise ConfigError(f"{where}mlp.kind {form!r} is not known (dense)")
            (ff,) = _sizes(mlp, ("ff",), where + "mlp.")
            mlp = DenseFeedForward(ff)
        return cls(kind, mixer, mlp)

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class PairTable:
    """Row (previous token * mul_prev + token * mul_cur) mod buckets of a second table is added
    to a token's embedding; a sequence's first token takes the row after the buckets."""

    buckets: int
    mul_prev: int
    mul_cur: int

    @classmethod
    def from_dict(cls, data, where):
        (buckets,) = _sizes(data, ("buckets",), where)
        factors = []
        for key in ("mul_prev", "mul_cur"):
            value = _need(data, key, where)
            if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                raise ConfigError(f"{where}{key} must be a non-negative integer, got {value!r}")
            factors.append(value)
        return cls(buckets, *factors)

    def to_dict(self):
        return {"buckets": self.buckets, "mul_cur": self.mul_cur, "mul_prev": self.mul_prev}


@dataclass(frozen=True)
class LamisunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram: PairTable | None
    taps: int | None
    layers: tuple[LamisunLayer, ...]
    extra: Mapping[str, Any] = field(default_factory=dict, repr=False)

    def __post_init__(self) -> None:
        positive_int("vocab", self.vocab)
        positive_int("width", self.width)
        positive("norm.eps", self.norm_eps)
        positive("embedding.scale", self.embedding_scale)
        if self.taps is not None:
            positive_int("canon.taps", self.taps)
        if not self.layers:
            raise ConfigError("layers is empty")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "LamisunConfig":
        name = data.get("architecture", data.get("model_type"))
        if str(name).lower() != NAME.lower():
            raise ConfigError(f"architecture {name!r} is not a {NAME} configuration")
        layers = _need(data, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("layers must be a list")
        embedding = data.get("embedding") or {}
        bigram = embedding.get("bigram")
        canon = data.get("canon")
        known = {"architecture", "model_type", "layers", "norm", "vocab", "width", "embedding",
                 "canon"}
        return cls(vocab=_need(data, "vocab", ""), width=_need(data, "width", ""),
                   norm_eps=float(_need(_need(data, "norm", ""), "eps", "norm.")),
                   embedding_scale=float(embedding.get("scale", 1.0)),
                   bigram=None if bigram is None
                   else PairTable.from_dict(bigram, "embedding.bigram."),
                   taps=None if canon is None else _need(canon, "taps", "canon."),
                   layers=tuple(LamisunLayer.from_dict(entry, f"layers[{i}].")
                                for i, entry in enumerate(layers)),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(self.extra)
        embedding: dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = self.bigram.to_dict()
        out.update(architecture=NAME, embedding=embedding,
                   layers=[layer.to_dict() for layer in self.layers],
                   norm={"eps": self.norm_eps}, vocab=self.vocab, width=self.width)
        if self.taps is not None:
            out["canon"] = {"taps": self.taps}
        return out
