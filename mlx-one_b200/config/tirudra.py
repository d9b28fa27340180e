"""Typed configuration of Tirudra, read from its config.json keys.

A Tirudra config.json has ``architecture`` ("Tirudra"), ``vocab``, ``width``, ``norm.eps``,
``logit_scale`` (a factor on the logits) and a list ``layers``. Every layer entry gives its
``type`` (the mixer it has), the mixer's sizes under ``mixer`` and its feed-forward under ``mlp``
(null: none; ``kind`` ``moe``: routed experts). The mixers:

``attention``: grouped-query softmax attention (``heads``, ``kv_heads``, ``dim``, ``vdim``,
``scale``) with a short causal convolution of ``conv`` taps on every channel of its queries,
keys and values, normed queries and keys, rotary positions (``rot``: ``base``, ``dims`` and an
optional ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``), a sliding window that
also keeps the sequence's first tokens (``mask``: ``size``, ``keep_first``) and a sigmoid gate on
every value of the heads' outputs.

``attention_2``: grouped-query softmax attention whose values are its keys as projected, with
biased projections, normed queries and keys, rotary positions (``scaling`` with ``factor``,
``low``, ``high``, ``original``), every earlier key visible, and one sigmoid gate per head.

``mamba2``: a selective state space (``heads``, ``vdim``, ``state``, ``groups``) behind a short
causal convolution of ``conv`` taps, gated and normed in ``norm_groups`` equal parts.

The routed feed-forward (``expert.ff``; ``router.experts``, ``router.top``, ``router.identity``:
outputs of the router beyond the experts that hand the input on as it is; ``shared.ff``: an
expert that every token uses, behind a sigmoid gate).

Nothing here has a default that stands for a size: a key that the design requires and that is
absent is an error with the key's path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .base import ConfigError, divisible, positive, positive_int

NAME = "Tirudra"


def _need(data: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(data, Mapping) or key not in data:
        raise ConfigError(f"{where}{key} is missing")
    return data[key]


def _count(data, key, where, least=0):
    value = _need(data, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"{where}{key} must be an integer of at least {least}, got {value!r}")
    return value


@dataclass(frozen=True)
class Rotary:
    """``scaling`` keeps the keys it was given: (factor, original, fast, slow) stretches the
    frequencies between two numbers of turns and scales cosine and sine; (factor, original, low,
    high) is the rule by wavelength."""

    base: float
    dims: int
    scaling: Mapping[str, float] | None = None

    FORMS = (("factor", "original", "fast", "slow"), ("factor", "original", "low", "high"))

    @classmethod
    def from_dict(cls, data, where, forms=None):
        dims = _need(data, "dims", where)
        positive_int(where + "dims", dims)
        if dims % 2:
            raise ConfigError(f"{where}dims ({dims}) must be even")
        base = float(_need(data, "base", where))
        positive(where + "base", base)
        scaling = data.get("scaling")
        if scaling is not None:
            form = next((keys for keys in (forms or cls.FORMS) if all(k in scaling for k in keys)), None)
            if form is None:
                wanted = " or ".join("(" + ", ".join(keys) + ")" for keys in (forms or cls.FORMS))
                raise ConfigError(f"{where}scaling must give {wanted}")
            scaling = {key: float(scaling[key]) for key in form}
            for key, value in scaling.items():
                positive(f"{where}scaling.{key}", value)
            if "low" in scaling and scaling["low"] == scaling["high"]:
                raise ConfigError(f"{where}scaling.high and {where}scaling.low must differ")
        return cls(base, dims, scaling)

    def to_dict(self):
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = {key: int(value) if key == "original" and float(value).is_integer()
                              else value for key, value in self.scaling.items()}
        return out


def _heads(data, where):
    heads, kv_heads = _need(data, "heads", where), _need(data, "kv_heads", where)
    divisible(where + "heads", heads, where + "kv_heads", kv_heads)
    dim, vdim = _need(data, "dim", where), _need(data, "vdim", where)
    positive_int(where + "dim", dim)
    positive_int(where + "vdim", vdim)
    scale = float(_need(data, "scale", where))
    positive(where + "scale", scale)
    return heads, kv_heads, dim, vdim, scale


def _rotary(data, where, dim, forms):
    rot = data.get("rot")
    rot = None if rot is None else Rotary.from_dict(rot, where + "rot.", forms)
    if rot is not None and rot.dims > dim:
        raise ConfigError(f"{where}rot.dims ({rot.dims}) exceeds {where}dim ({dim})")
    return rot


@dataclass(frozen=True)
class ConvAttentionMixer:
    """Heads, sizes, score scale, taps of the convolutions (None: none), window and how many
    first tokens stay visible behind it (window None: every earlier key), rotation."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int | None
    window: int | None
    keep_first: int
    rot: Rotary | None

    @classmethod
    def from_dict(cls, data, where):
        heads, kv_heads, dim, vdim, scale = _heads(data, where)
        conv = data.get("conv")
        if conv is not None:
            positive_int(where + "conv", conv)
        window, keep_first = None, 0
        if data.get("mask") is not None:
            window = _need(data["mask"], "size", where + "mask.")
            positive_int(where + "mask.size", window)
            if data["mask"].get("keep_first") is not None:
                keep_first = _count(data["mask"], "keep_first", where + "mask.")
        return cls(heads, kv_heads, dim, vdim, scale, conv, window, keep_first,
                   _rotary(data, where, dim, Rotary.FORMS[:1]))

    def to_dict(self):
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                               "scale": self.scale, "vdim": self.vdim}
        if self.conv is not None:
            out["conv"] = self.conv
        if self.window is not None:
            out["mask"] = {"keep_first": self.keep_first, "size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class SharedKeyValueMixer:
    """Heads, the size of a head (keys are the values, so both sizes are one), score scale,
    rotation."""

    heads: int
    kv_heads: int
    dim: int
    scale: float
    rot: Rotary | None

    @classmethod
    def from_dict(cls, data, where):
        heads, kv_heads, dim, vdim, scale = _heads(data, where)
        if vdim != dim:
            raise ConfigError(f"{where}vdim ({vdim}) must equal {where}dim ({dim}): the values "
                              "are the keys")
        return cls(heads, kv_heads, dim, scale, _rotary(data, where, dim, Rotary.FORMS[1:]))

    def to_dict(self):
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                               "scale": self.scale, "vdim": self.dim}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class StateSpaceMixer:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, data, where):
        for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
            positive_int(where + key, _need(data, key, where))
        divisible(where + "heads", data["heads"], where + "groups", data["groups"])
        inner = data["heads"] * data["vdim"]
        if inner % data["norm_groups"]:
            raise ConfigError(f"{where}heads * {where}vdim ({inner}) must be divisible by "
                              f"{where}norm_groups ({data['norm_groups']})")
        return cls(data["heads"], data["vdim"], data["state"], data["groups"], data["conv"],
                   data["norm_groups"])

    def to_dict(self):
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads,
                "norm_groups": self.norm_groups, "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class RoutedFeedForward:
    """``experts`` feed-forwards of width ``ff`` and ``identity`` further outputs of the router
    that hand the input on; a token uses ``top`` of them all; a shared expert of width
    ``shared_ff`` (None: none)."""

    ff: int
    experts: int
    top: int
    identity: int
    shared_ff: int | None

    @classmethod
    def from_dict(cls, data, where):
        ff = _need(_need(data, "expert", where), "ff", where + "expert.")
        positive_int(where + "expert.ff", ff)
        router = _need(data, "router", where)
        experts = _need(router, "experts", where + "router.")
        top = _need(router, "top", where + "router.")
        positive_int(where + "router.experts", experts)
        positive_int(where + "router.top", top)
        identity = 0
        if router.get("identity") is not None:
            identity = _count(router, "identity", where + "router.")
        if top > experts + identity:
            raise ConfigError(f"{where}router.top ({top}) exceeds the router's outputs "
                              f"({experts + identity})")
        shared_ff = None
        if data.get("shared") is not None:
            shared_ff = _need(data["shared"], "ff", where + "shared.")
            positive_int(where + "shared.ff", shared_ff)
        return cls(ff, experts, top, identity, shared_ff)

    def to_dict(self):
        out: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe",
                               "router": {"experts": self.experts, "identity": self.identity,
                                          "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXERS = {"attention": ConvAttentionMixer, "attention_2": SharedKeyValueMixer,
          "mamba2": StateSpaceMixer}


@dataclass(frozen=True)
class TirudraLayer:
    type: str
    mixer: Any
    mlp: RoutedFeedForward | None

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
            if form != "moe":
                raise ConfigError(f"{where}mlp.kind {form!r} is not known (moe)")
            mlp = RoutedFeedForward.from_dict(mlp, where + "mlp.")
        return cls(kind, mixer, mlp)

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict(), "type": self.type}


@dataclass(frozen=True)
class TirudraConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: tuple[TirudraLayer, ...]
    extra: Mapping[str, Any] = field(default_factory=dict, repr=False)

    def __post_init__(self) -> None:
        positive_int("vocab", self.vocab)
        positive_int("width", self.width)
        positive("norm.eps", self.norm_eps)
        positive("logit_scale", self.logit_scale)
        if not self.layers:
            raise ConfigError("layers is empty")

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "TirudraConfig":
        name = data.get("architecture", data.get("model_type"))
        if str(name).lower() != NAME.lower():
            raise ConfigError(f"architecture {name!r} is not a {NAME} configuration")
        layers = _need(data, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("layers must be a list")
        known = {"architecture", "model_type", "layers", "norm", "vocab", "width", "logit_scale"}
        return cls(vocab=_need(data, "vocab", ""), width=_need(data, "width", ""),
                   norm_eps=float(_need(_need(data, "norm", ""), "eps", "norm.")),
                   logit_scale=float(data.get("logit_scale", 1.0)),
                   layers=tuple(TirudraLayer.from_dict(entry, f"layers[{i}].")
                                for i, entry in enumerate(layers)),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(self.extra)
        out.update(architecture=NAME, layers=[layer.to_dict() for layer in self.layers],
                   logit_scale=self.logit_scale, norm={"eps": self.norm_eps}, vocab=self.vocab,
                   width=self.width)
        return out
