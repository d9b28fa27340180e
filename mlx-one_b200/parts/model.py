"""A model built from a ``ModelSpec`` and a set of tensors."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .base import Runtime, StepContext
from .registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, MIXERS, NORMS
from .spec import LayerCall, ModelSpec, PartSpec, TensorSpec


def _part_tensors(registry, spec: PartSpec, prefix: str) -> dict[str, TensorSpec]:
    cls = registry.get(spec.kind)
    return {prefix + spec.stored_name(local): t for local, t in cls.tensors(spec).items()}


def expected_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """Every stored tensor of the model by full name: the weight contract."""
    out = {spec.embedding: TensorSpec((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for registry, part in ((BLOCKS, layer.block), (MIXERS, layer.mixer),
                               (NORMS, layer.mixer_norm), (FEED_FORWARDS, layer.feed_forward),
                               (NORMS, layer.feed_forward_norm)):
            if part is not None:
                out.update(_part_tensors(registry, part, layer.prefix))
    out.update(_part_tensors(NORMS, spec.final_norm, ""))
    if spec.embedding_part is not None:
        out.update(_part_tensors(EMBEDDINGS, spec.embedding_part, ""))
    out.update(spec.vectors)
    if spec.head is not None:
        out[spec.head] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return out


def entry_key(entry: int, name: str | None = None):
    """The key of a cache entry: the entry's number, or (number, name) for one of the several
    things that a mixer made of several mixers keeps."""
    return entry if name is None else (entry, name)


# what a block keeps for itself is stored beside its mixer's cache, under names that begin so
BLOCK_PREFIX = "block:"
# the cache entry of the embedding part
EMBEDDING_ENTRY = (-1, "embedding")


def _needs_of(spec: ModelSpec, call: LayerCall, index: int) -> dict[Any, Any]:
    entry = index if call.cache is None else call.cache
    layer = spec.layers[call.layer]
    out: dict[Any, Any] = {}
    own = BLOCKS.get(layer.block.kind).cache_need(layer.block)
    for name, part in (own or {}).items():
        if part is not None:
            out[entry_key(entry, BLOCK_PREFIX + name)] = part
    need = MIXERS.get(layer.mixer.kind).cache_need(layer.mixer)
    if need is None:
        return out
    if isinstance(need, Mapping):
        out.update({entry_key(entry, name): part for name, part in need.items()
                    if part is not None})
    else:
        out[entry] = need
    return out


def cache_entries(spec: ModelSpec) -> dict[Any, Any]:
    """Cache entry -> need, for every entry that a call of the order writes. A mixer whose
    ``cache_need`` is a mapping name -> need (several mixers side by side) has one entry per
    name, keyed (entry, name)."""
    needs: dict[Any, Any] = {}
    for index, call in enumerate(spec.order):
        if not call.writes_cache:
            continue
        for key, need in _needs_of(spec, call, index).items():
            if key in needs and needs[key] != need:
                raise ValueError(f"cache entry {key} is written with two different needs")
            needs[key] = need
    for index, call in enumerate(spec.order):
        if call.writes_cache:
            continue
        for key, need in _needs_of(spec, call, index).items():
            if key not in needs:
                raise ValueError(f"call {index} reads cache entry {key} that nothing writes")
            if needs[key] != need:
                raise ValueError(f"call {index} reads cache entry {key} of another shape")
    if spec.embedding_part is not None:
        need = EMBEDDINGS.get(spec.embedding_part.kind).cache_need(spec.embedding_part)
        if need is not None:
            needs[EMBEDDING_ENTRY] = need
    return needs


def view_of(views: Mapping[Any, Any], entry: int):
    """What a call's mixer gets as ``cache``: the entry's view, or for a mixer of several
    mixers a dict name -> view."""
    if entry in views:
        return views[entry]
    named = {key[1]: view for key, view in views.items()
             if isinstance(key, tuple) and key[0] == entry and not key[1].startswith(BLOCK_PREFIX)}
    return named or None


def block_view_of(views: Mapping[Any, Any], entry: int):
    """What a call's block gets as ``own_cache``: a dict name -> view of what it keeps itself."""
    return {key[1][len(BLOCK_PREFIX):]: view for key, view in views.items()
            if isinstance(key, tuple) and key[0] == entry and key[1].startswith(BLOCK_PREFIX)}


class Model:
    """Embedding, layers in the spec's order, final norm and output matrix.

    ``forward(ctx)`` runs the tokens of a step and returns the 32-bit residual stream with
    the last block's output still pending; ``logits(residual, delta, rows)`` norms the
    wanted rows and multiplies them with the output matrix."""

    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor],
                 runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime
        self.ops = runtime.ops

        def build(registry, part: PartSpec, prefix: str, **extra):
            cls = registry.get(part.kind)
            local = {name: tensors[prefix + part.stored_name(name)]
                     for name in cls.tensors(part)}
            return cls(part, local, runtime, **extra)

        self.embedding = tensors[spec.embedding].to(runtime.dtype).contiguous()
        self.embedding_part = None
        if spec.embedding_part is not None:
            self.embedding_part = build(EMBEDDINGS, spec.embedding_part, "")
            self.embedding = self.embedding_part.table
        self.layers = []
        for layer in spec.layers:
            roles = dict(
                mixer=build(MIXERS, layer.mixer, layer.prefix),
                mixer_norm=build(NORMS, layer.mixer_norm, layer.prefix),
                feed_forward=None if layer.feed_forward is None
                else build(FEED_FORWARDS, layer.feed_forward, layer.prefix),
                feed_forward_norm=None if layer.feed_forward_norm is None
                else build(NORMS, layer.feed_forward_norm, layer.prefix),
            )
            self.layers.append(build(BLOCKS, layer.block, layer.prefix, **roles))
        self.final_norm = build(NORMS, spec.final_norm, "")
        self.head = (self.embedding if spec.head is None
                     else tensors[spec.head].to(runtime.dtype).contiguous())
        self.order = tuple(
            LayerCall(call.layer, index if call.cache is None else call.cache, call.writes_cache,
                      call.inject)
            for index, call in enumerate(spec.order))
        # what is added to the stream before a call: one 32-bit row per injection
        self.injected = {}
        for index, call in enumerate(spec.order):
            if call.inject is not None and call.inject.vector is not None:
                rows = tensors[call.inject.vector]
                if not 0 <= call.inject.row < rows.shape[0]:
                    raise ValueError(f"{call.inject.vector} has no row {call.inject.row}")
                self.injected[index] = rows[call.inject.row].to(torch.float32).contiguous()
        # a matrix applied to the stream and the embeddings side by side before a call
        self.mixing = {}
        for index, call in enumerate(spec.order):
            if call.inject is not None and call.inject.mix is not None:
                matrix = tensors[call.inject.mix]
                if tuple(matrix.shape) != (spec.hidden_size, 2 * spec.hidden_size):
                    raise ValueError(f"{call.inject.mix} has shape {tuple(matrix.shape)}, expected "
                                     f"{(spec.hidden_size, 2 * spec.hidden_size)}")
                if call.inject.mix not in self.mixing:
                    self.mixing[call.inject.mix] = matrix.to(runtime.dtype).contiguous()
        self.softcap = None if spec.logit_softcap is None else float(spec.logit_softcap)
        self.logit_scale = float(spec.logit_scale)
        # the factor with which the pending output of the last forward is still to be added
        self.pending_scale = 1.0
        self.cache_needs = cache_entries(spec)
        # whether steps of this model may be captured as CUDA graphs: every part says so
        parts = [self.final_norm]
        for block in self.layers:
            parts += [part for part in (block, block.mixer, block.mixer_norm, block.feed_forward,
                                        block.feed_forward_norm) if part is not None]
            parts += list(getattr(block.mixer, "inner_parts", lambda: ())())
        if self.embedding_part is not None:
            parts.append(self.embedding_part)
        self.capturable = all(getattr(part, "capturable", True) for part in parts)
        # blocks that read the streams of the calls before them (see Block.keeps_streams)
        self.keeps_streams = any(block.keeps_streams for block in self.layers)
        self.own_caches = [bool(type(block).cache_need(block.spec)) for block in self.layers]
        # For debugging: called as observer(place, residual, delta) after the embedding
        # (place -1) and after every call of a layer (place = its number in the order); the
        # hidden state there is residual + s * delta, s the block's ``pending_scale`` (1 unless the
        # architecture gives its parts' outputs a factor). It sees the step's own tensors (a step's
        # rows may be followed by fillers): copy what is to be kept. Steps that are replayed from
        # a CUDA graph do not call it.
        self.observer = None

    def forward(self, ctx: StepContext):
        kept = None
        if self.keeps_streams:
            # the embedding's output, every call's result, and what the last call passes on
            kept = torch.empty((len(self.order) + 2, ctx.tokens, self.spec.hidden_size),
                               dtype=torch.float32, device=self.runtime.device)
        if self.embedding_part is not None:
            residual = self.embedding_part.forward(
                ctx, ctx.views.get(EMBEDDING_ENTRY), None if kept is None else kept[0])
        else:
            residual = self.ops.embedding(ctx.token_ids, self.embedding)
            if kept is not None:
                kept[0].copy_(residual)
        if kept is not None:
            # the first call works on a copy: the embedding's output is read again later
            residual = self.ops.stream_average(kept, None, 1, kept[1])
        delta, scale = None, 1.0
        if self.observer is not None:
            self.observer(-1, residual, delta)
        for place, call in enumerate(self.order):
            extra = {} if delta is None or scale == 1.0 else {"delta_scale": scale}
            if call.inject is not None and call.inject.mix is not None:
                # the stream (with the pending output) and the token's embedding side by side in
                # the compute dtype, one product back into a 32-bit stream, the pass's vector as
                # the product's bias
                both = self.ops.concat_stream(residual, delta, ctx.token_ids, self.embedding,
                                              self.runtime.dtype, **extra)
                residual = self.ops.linear(both, self.mixing[call.inject.mix],
                                           self.injected.get(place), out_dtype=torch.float32)
                delta, extra = None, {}
            elif call.inject is not None:
                # the pending output, the token's embedding once more and the pass's vector
                # enter the 32-bit stream in one kernel
                self.ops.add_vectors(residual, delta, ctx.token_ids,
                                     self.embedding if call.inject.embedding else None,
                                     self.injected.get(place), **extra)
                delta, extra = None, {}
            block = self.layers[call.layer]
            if self.own_caches[call.layer]:
                extra["own_cache"] = block_view_of(ctx.views, call.cache)
            if block.keeps_streams:
                residual, delta = block.forward(
                    residual, delta, ctx, view_of(ctx.views, call.cache), call.writes_cache,
                    streams=(kept, place), **extra)
            else:
                delta = block.forward(residual, delta, ctx, view_of(ctx.views, call.cache),
                                      call.writes_cache, **extra)
                if kept is not None:
                    raise ValueError("a model that keeps its streams has blocks that all do")
            scale = block.pending_scale
            if self.observer is not None:
                self.observer(place, residual, delta)
        self.pending_scale = 1.0 if delta is None else scale
        return residual, delta

    def logits(self, residual, delta, rows: torch.Tensor | None) -> torch.Tensor:
        """32-bit logits [len(rows), vocab] at the token rows ``rows`` (int32, device); None:
        at every row, in order (a step of single tokens that all want theirs: nothing to pick)."""
        if rows is None:
            picked, picked_delta = residual, delta
        else:
            picked, picked_delta = self.ops.gather_rows(residual, delta, rows)
        # the output product may apply the norm itself where the kernels can do that
        extra = {}
        if picked_delta is not None and self.pending_scale != 1.0:
            extra["delta_scale"] = self.pending_scale
        if self.final_norm.supports_lazy:
            normed = self.final_norm.forward(picked, picked_delta, lazy=True, **extra)
        else:
            normed = self.final_norm.forward(picked, picked_delta, **extra)
        logits = self.ops.linear(normed, self.head, out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            self.ops.scale_values(logits, self.logit_scale)
        if self.softcap is not None:
            self.ops.softcap(logits, self.softcap)
        return logits

    def weight_bytes(self) -> int:
        """Bytes of every matrix and vector a step reads once (a tied table counts once)."""
        seen, total = set(), 0
        def visit(obj):
            nonlocal total
            for value in vars(obj).values():
                if isinstance(value, torch.Tensor):
                    key = value.data_ptr()
                    if key not in seen:
                        seen.add(key)
                        total += value.numel() * value.element_size()
                elif hasattr(value, "spec") and hasattr(value, "runtime"):
                    visit(value)
                elif isinstance(value, (list, tuple)):
                    for item in value:
                        if isinstance(item, torch.Tensor):
                            if item.data_ptr() not in seen:
                                seen.add(item.data_ptr())
                                total += item.numel() * item.element_size()
                        elif hasattr(item, "spec") and hasattr(item, "runtime"):
                            visit(item)
        for layer in self.layers:
            visit(layer)
        visit(self.final_norm)
        for matrix in self.mixing.values():
            if matrix.data_ptr() not in seen:
                seen.add(matrix.data_ptr())
                total += matrix.numel() * matrix.element_size()
        if self.head.data_ptr() not in seen:
            total += self.head.numel() * self.head.element_size()
        return total
