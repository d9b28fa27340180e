"""Lamisun described in parts.

The stream starts as the token's embedding times a scale plus a row of a second table chosen by
a hash of the token and the one before it. Every layer adds its parts' normed outputs:
x <- x + norm1(mixer(in(x))), x <- x + norm2(feed_forward(in(x))), where in(x) = x + a causal
convolution of x over time on every channel. After layer i the stream that goes on is a stored
weighting of the embedding's output and the results of the layers 0 .. i. The mixer of a layer
is either attention over one latent row per token (a rotated key part shared by all heads,
neighbouring dimensions paired; a sigmoid output gate) or differential attention (two score
maps per head, normed queries and keys, no rotation, chunks of positions that see only
themselves). The feed-forward is down(xielu(up x)) with two stored numbers that shape the
activation, or absent.

Stored names: ``embed``, ``bigram``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.canon1``, ``l<i>.canon2``, ``l<i>.dwa``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,
g,o}`` (latent attention) or ``l<i>.mix.{q,k,v,q.norm,k.norm,lq1,lk1,lq2,lk2,o}`` (differential
attention), ``l<i>.mlp.{up,down,act}``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.lamisun import DifferentialMixer, LamisunConfig, LatentMixer
from ..config.registry import Architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _latent(mixer: LatentMixer, width: int, eps: float) -> PartSpec:
    position = PartSpec("rope_long", {"theta": mixer.rot.base, "rotary_dim": mixer.rot.dims,
                                      "layout": "neighbours", "factor": None})
    return PartSpec("latent_attention", {
        "hidden": width, "heads": mixer.heads, "head_dim": mixer.dim, "rot_dim": mixer.rot_dim,
        "value_dim": mixer.vdim, "latent": mixer.kv_rank, "eps": eps, "position": position,
        "scale": mixer.scale, "gate": True,
    }, "mix.", {"down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g",
                "out": "o"})


def _differential(mixer: DifferentialMixer, width: int, eps: float) -> PartSpec:
    return PartSpec("differential_attention", {
        "hidden": width, "heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim,
        "value_dim": mixer.vdim, "eps": eps, "scale": mixer.scale, "diff": mixer.diff,
        "chunk": mixer.chunk,
    }, "mix.", {"q_norm": "q.norm", "k_norm": "k.norm", "out": "o"})


def describe(config: LamisunConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"size": width, "eps": eps}, "", {"weight": name})
    layers = []
    for index, layer in enumerate(config.layers):
        if isinstance(layer.mixer, LatentMixer):
            mixer = _latent(layer.mixer, width, eps)
        else:
            mixer = _differential(layer.mixer, width, eps)
        feed_forward = feed_forward_norm = None
        if layer.mlp is not None:
            feed_forward = PartSpec("dense", {"hidden": width, "width": layer.mlp.ff,
                                              "activation": "xielu"}, "mlp.",
                                    {"up.weight": "up", "down.weight": "down"})
            feed_forward_norm = norm("norm2")
        block = PartSpec("outnorm", {"hidden": width, "taps": config.taps, "streams": index + 2,
                                     "feed_forward": layer.mlp is not None}, "",
                         {"conv1": "canon1", "conv2": "canon2", "average": "dwa"})
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=mixer,
                                mixer_norm=norm("norm1"), feed_forward=feed_forward,
                                feed_forward_norm=feed_forward_norm))
    if config.bigram is None:
        embedding = PartSpec("table", {"vocab": config.vocab, "hidden": width,
                                       "scale": config.embedding_scale}, "", {"table": "embed"})
    else:
        embedding = PartSpec("pair_hash", {
            "vocab": config.vocab, "hidden": width, "scale": config.embedding_scale,
            "buckets": config.bigram.buckets, "mul_prev": config.bigram.mul_prev,
            "mul_cur": config.bigram.mul_cur}, "", {"table": "embed", "pairs": "bigram"})
    return ModelSpec(
        architecture="lamisun", vocab_size=config.vocab, hidden_size=width, embedding="embed",
        layers=tuple(layers), order=tuple(LayerCall(index) for index in range(len(layers))),
        final_norm=norm("final.norm"), head="head", max_positions=1 << 30,
        embedding_part=embedding)


ARCHITECTURE = Architecture("lamisun", LamisunConfig, describe)
