"""Tirudra described in parts.

Every layer norms its parts' inputs and their outputs: x <- x + norm1b(mixer(norm1(x))), then
x <- x + norm2b(feed_forward(norm2(x))); the norms' weights are stored around zero. The mixer
of a layer is one of three. ``attention``: grouped-query softmax attention whose queries, keys
and values pass a short causal convolution over time right after their projections, with normed
queries and keys, rotary positions on the first dimensions of a head (halves paired,
frequencies stretched between two numbers of turns, cosine and sine scaled), a sliding window
behind which the sequence's first tokens stay visible, and a sigmoid gate on every value of the
heads' outputs. ``attention_2``: grouped-query softmax attention with biased query and key
projections whose values are the keys as projected, normed queries and keys, rotary positions
with the long-context rule by wavelength, every earlier key visible, one sigmoid gate per head.
``mamba2``: a selective state space with a 32-bit matrix state per head behind a short causal
convolution, gated and normed in groups. The feed-forward is a mixture of routed experts:
softmax scores, a stored correction that enters the choice only, weights that are not
renormalised, outputs of the router that stand for the input itself, and a shared expert behind
a sigmoid gate; or absent. The logits are multiplied by a constant.

Stored names: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1``, ``norm1b``,
``norm2``, ``norm2b``; ``l<i>.mix.{q,k,v,g,o}``, ``.q.norm``, ``.k.norm``, ``.{q,k,v}.conv``
(attention); ``l<i>.mix.{q,k,g,o}``, ``.q.b``, ``.k.b``, ``.q.norm``, ``.k.norm`` (attention_2);
``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}`` (mamba2); ``l<i>.mlp.router``,
``.correction``, ``.e<j>.{gate,up,down}``, ``.shared.{gate,up,down,sg}``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.registry import Architecture
from ..config.tirudra import (ConvAttentionMixer, RoutedFeedForward, SharedKeyValueMixer,
                              StateSpaceMixer, TirudraConfig)
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                    "out_proj.weight": "o", "q_proj.bias": "q.b", "k_proj.bias": "k.b",
                    "q_layernorm.weight": "q.norm", "k_layernorm.weight": "k.norm",
                    "gate.weight": "g", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}


def _position(rot) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    scaling = rot.scaling or {}
    if "low" in scaling:
        return PartSpec("rope_long", {"theta": rot.base, "rotary_dim": rot.dims, "layout": "halves",
                                      **{key: scaling[key] for key in ("factor", "original", "low", "high")}})
    return PartSpec("yarn", {"theta": rot.base, "rotary_dim": rot.dims,
                             **{key: scaling.get(key) for key in ("factor", "original", "fast", "slow")}})


def _conv_attention(mixer: ConvAttentionMixer, width: int, eps: float) -> PartSpec:
    return PartSpec("attention", {
        "hidden": width, "heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim,
        "value_dim": mixer.vdim, "bias": False, "qk_norm_eps": eps, "qk_norm": "weighted_before",
        "position": _position(mixer.rot), "scale": mixer.scale, "window": mixer.window,
        "keep_first": mixer.keep_first if mixer.window is not None else 0,
        "conv_taps": mixer.conv, "gate": "values"}, "mix.", _ATTENTION_NAMES)


def _shared_key_value_attention(mixer: SharedKeyValueMixer, width: int, eps: float) -> PartSpec:
    return PartSpec("attention", {
        "hidden": width, "heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim,
        "value_dim": mixer.dim, "bias": True, "values": "keys", "qk_norm_eps": eps,
        "qk_norm": "weighted_before", "position": _position(mixer.rot), "scale": mixer.scale,
        "window": None, "gate": "heads"}, "mix.", _ATTENTION_NAMES)


def _state_space(mixer: StateSpaceMixer, width: int, eps: float) -> PartSpec:
    return PartSpec("mamba2", {
        "hidden": width, "heads": mixer.heads, "value_dim": mixer.vdim, "state": mixer.state,
        "groups": mixer.groups, "taps": mixer.conv, "norm_groups": mixer.norm_groups, "eps": eps},
        "mix.", {"conv_bias": "conv.b"})


def _feed_forward(mlp: RoutedFeedForward, width: int) -> PartSpec:
    return PartSpec("routed", {
        "hidden": width, "width": mlp.ff, "experts": mlp.experts, "top": mlp.top,
        "identity": mlp.identity, "shared_width": mlp.shared_ff, "activation": "silu",
        "scores": "softmax", "correction": True, "normalize": False,
        "shared_gate": mlp.shared_ff is not None}, "mlp.")


def describe(config: TirudraConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"size": width, "eps": eps, "offset": 1.0}, "",
                                 {"weight": name})
    layers = []
    for index, layer in enumerate(config.layers):
        if isinstance(layer.mixer, ConvAttentionMixer):
            mixer = _conv_attention(layer.mixer, width, eps)
        elif isinstance(layer.mixer, SharedKeyValueMixer):
            mixer = _shared_key_value_attention(layer.mixer, width, eps)
        else:
            assert isinstance(layer.mixer, StateSpaceMixer)
            mixer = _state_space(layer.mixer, width, eps)
        feed_forward = feed_forward_norm = None
        if layer.mlp is not None:
            feed_forward = _feed_forward(layer.mlp, width)
            feed_forward_norm = norm("norm2")
        block = PartSpec("sandwich", {"size": width, "eps": eps, "offset": 1.0,
                                      "feed_forward": layer.mlp is not None}, "",
                         {"post_mixer": "norm1b", "post_feed_forward": "norm2b"})
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=mixer,
                                mixer_norm=norm("norm1"), feed_forward=feed_forward,
                                feed_forward_norm=feed_forward_norm))
    return ModelSpec(
        architecture="tirudra", vocab_size=config.vocab, hidden_size=width, embedding="embed",
        layers=tuple(layers), order=tuple(LayerCall(index) for index in range(len(layers))),
        final_norm=norm("final.norm"), head="head", max_positions=1 << 30,
        logit_scale=config.logit_scale)


ARCHITECTURE = Architecture("tirudra", TirudraConfig, describe)
