"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import Block, FixedState
from .registry import BLOCKS
from .spec import TensorSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """h = x + mixer(norm(x)); out = h + feed_forward(norm(h)). Each residual add is fused
    with the norm that follows it, so the block returns its last output unadded; a part that
    ``fuses_residual`` may instead add its output into the stream itself and return None.
    A layer without a feed-forward ends after the mixer. Parameter ``residual_scale`` (1): the
    factor m in h = x + m mixer(norm(x)); out = h + m feed_forward(norm(h)). The factor is
    applied where the output is added: by the part itself if it adds into the stream and
    ``scales_residual``, else by the norm that follows (``delta_scale``).
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:160-179."""

    def __init__(self, spec, tensors, runtime, **roles):
        super().__init__(spec, tensors, runtime, **roles)
        self.scale = float(spec.get("residual_scale", 1.0))
        self.pending_scale = self.scale
        for part in (self.mixer, self.feed_forward):
            if part is not None:
                part.residual_scale = self.scale

    @staticmethod
    def _norm(norm, residual, delta, consumer, scale=1.0):
        extra = {} if scale == 1.0 else {"delta_scale": scale}
        if consumer.accepts_normed_input and norm.supports_lazy:
            return norm.forward(residual, delta, lazy=True, **extra)
        return norm.forward(residual, delta, **extra)

    def _fuses(self, part):
        return part.fuses_residual and (self.scale == 1.0 or part.scales_residual)

    def forward(self, residual, delta, ctx, cache, write, delta_scale=1.0):
        normed = self._norm(self.mixer_norm, residual, delta, self.mixer, delta_scale)
        if self._fuses(self.mixer):
            mixed = self.mixer.forward(normed, ctx, cache, write, residual=residual)
        else:
            mixed = self.mixer.forward(normed, ctx, cache, write)
        if self.feed_forward is None:
            return mixed
        normed = self._norm(self.feed_forward_norm, residual, mixed, self.feed_forward, self.scale)
        if self._fuses(self.feed_forward):
            return self.feed_forward.forward(normed, ctx, residual=residual)
        return self.feed_forward.forward(normed, ctx)


@BLOCKS.register("outnorm")
class OutputNormBlock(Block):
    """x <- x + norm1(mixer(in1(x))); x <- x + norm2(feed_forward(in2(x))): the norms are applied
    to the parts' outputs, the parts read the stream itself (rounded to the compute dtype).
    A layer without a feed-forward ends after the mixer. Parameters:

    ``taps`` (None: in(x) = x): in(x) = x + conv(x), a causal convolution over time on every
    channel of the 32-bit stream, conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j) with nothing
    before a sequence's start; ``conv1`` and ``conv2`` [hidden, taps] are the two sublayers'
    weights. The last taps - 1 rows of x that each sublayer read are kept per request in 32-bit.

    ``streams`` (None: the layer's result goes on as it is): the number n of streams that are
    averaged after the layer, with the stored weights ``average`` [n]: what the next layer reads
    is sum_j average[j] X_j, X_0 the embedding's output and X_(j+1) the result of the call j of
    the order (before any averaging), so n is this call's number plus two."""

    @classmethod
    def tensors(cls, spec):
        out = {}
        if spec.get("taps"):
            out["conv1"] = TensorSpec((spec["hidden"], spec["taps"]), "wide")
            if spec.get("feed_forward", True):
                out["conv2"] = TensorSpec((spec["hidden"], spec["taps"]), "wide")
        if spec.get("streams"):
            out["average"] = TensorSpec((spec["streams"],), "wide")
        return out

    @classmethod
    def cache_need(cls, spec):
        taps = spec.get("taps")
        if not taps or taps < 2:
            return None
        sublayers = 2 if spec.get("feed_forward", True) else 1
        return {"inputs": FixedState((sublayers, taps - 1, spec["hidden"]), "float32")}

    def __init__(self, spec, tensors, runtime, **roles):
        super().__init__(spec, tensors, runtime, **roles)
        self.taps = spec.get("taps") or 0
        self.conv1 = self.vector(tensors["conv1"]) if "conv1" in tensors else None
        self.conv2 = self.vector(tensors["conv2"]) if "conv2" in tensors else None
        self.average = self.vector(tensors["average"]) if "average" in tensors else None
        self.keeps_streams = self.average is not None
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("this block needs norms that can be applied to a part's output")

    def _read(self, residual, kernel, ctx, own_cache, write, sublayer):
        """What a sublayer reads: the stream (plus its convolution over time) in the compute dtype."""
        view = (own_cache or {}).get("inputs")
        return self.ops.stream_conv(residual, kernel, taps=self.taps, ctx=ctx, view=view,
                                    sublayer=sublayer, write=write, dtype=self.runtime.dtype)

    def forward(self, residual, delta, ctx, cache, write, own_cache=None, streams=None,
                delta_scale=1.0):
        if delta is not None:
            raise ValueError("this block takes a stream with nothing pending")
        mixed = self.mixer.forward(self._read(residual, self.conv1, ctx, own_cache, write, 0),
                                   ctx, cache, write)
        self.mixer_norm.add_normed(residual, mixed)
        if self.feed_forward is not None:
            out = self.feed_forward.forward(
                self._read(residual, self.conv2, ctx, own_cache, write, 1), ctx)
            self.feed_forward_norm.add_normed(residual, out)
        if self.average is None:
            return None
        kept, place = streams
        if self.average.numel() != place + 2:
            raise ValueError(f"call {place} of the order averages {place + 2} streams, "
                             f"{self.average.numel()} weights are stored")
        return self.ops.stream_average(kept, self.average, place + 2, kept[place + 2]), None


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """x <- x + post1(mixer(norm1(x))); x <- x + post2(feed_forward(norm2(x))): every part reads
    the normed stream and its output is normed once more before it is added. The norms ahead of
    the parts are the layer's ``mixer_norm`` and ``feed_forward_norm``; the norms behind them are
    the block's own: v / rms(v) * (offset + weight) over the model width, with the stored weights
    ``post_mixer`` and ``post_feed_forward``, taken and added in 32-bit. A layer without a
    feed-forward ends after the mixer. Parameters: ``size``, ``eps``, ``offset`` (0; 1 for
    weights stored around zero), ``feed_forward`` (True: the layer has one)."""

    @classmethod
    def tensors(cls, spec):
        init = "norm0" if spec.get("offset") else "norm"
        out = {"post_mixer": TensorSpec((spec["size"],), init)}
        if spec.get("feed_forward", True):
            out["post_feed_forward"] = TensorSpec((spec["size"],), init)
        return out

    def __init__(self, spec, tensors, runtime, **roles):
        super().__init__(spec, tensors, runtime, **roles)
        self.eps = float(spec["eps"])
        offset = float(spec.get("offset") or 0.0)
        weight = lambda name: (self.vector(tensors[name]) + offset).contiguous()
        self.post_mixer = weight("post_mixer")
        self.post_feed_forward = weight("post_feed_forward") if "post_feed_forward" in tensors else None
        if (self.feed_forward is None) != (self.post_feed_forward is None):
            raise ValueError("a feed-forward and the norm behind it come together")

    def _read(self, norm, residual, delta, consumer, scale=1.0):
        extra = {} if scale == 1.0 else {"delta_scale": scale}
        if delta is None and consumer.accepts_normed_input and norm.supports_lazy:
            return norm.forward(residual, delta, lazy=True, **extra)
        return norm.forward(residual, delta, **extra)

    def forward(self, residual, delta, ctx, cache, write, delta_scale=1.0):
        normed = self._read(self.mixer_norm, residual, delta, self.mixer, delta_scale)
        mixed = self.mixer.forward(normed, ctx, cache, write)
        self.ops.normed_mean_add(residual, [mixed], [self.post_mixer], self.eps)
        if self.feed_forward is not None:
            normed = self._read(self.feed_forward_norm, residual, None, self.feed_forward)
            out = self.feed_forward.forward(normed, ctx)
            self.ops.normed_mean_add(residual, [out], [self.post_feed_forward], self.eps)
        return None
