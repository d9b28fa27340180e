"""Embedding parts: what turns a step's token ids into the 32-bit stream."""

from __future__ import annotations

from .base import Embedding, FixedState
from .registry import EMBEDDINGS
from .spec import TensorSpec


@EMBEDDINGS.register("table")
class TableEmbedding(Embedding):
    """Row ``token`` of the table [vocab, hidden], times ``scale`` (1). Parameters: ``vocab``,
    ``hidden``, ``scale``."""

    @classmethod
    def tensors(cls, spec):
        return {"table": TensorSpec((spec["vocab"], spec["hidden"]))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.table = self.matrix(tensors["table"])
        self.scale = float(spec.get("scale", 1.0))

    def forward(self, ctx, cache, out=None):
        return self.ops.embedding_pairs(ctx.token_ids, self.table, self.scale, None, rule=None,
                                        ctx=ctx, view=None, out=out)


@EMBEDDINGS.register("pair_hash")
class PairHashEmbedding(TableEmbedding):
    """The table's row times ``scale``, plus a row of a second table ``pairs`` [buckets + 1,
    hidden] chosen by the token and the one before it in its sequence: row (previous * mul_prev +
    token * mul_cur) mod buckets, and row ``buckets`` for a sequence's first token. Parameters:
    ``vocab``, ``hidden``, ``scale``, ``buckets``, ``mul_prev``, ``mul_cur``. The token before a
    step's first one is kept per request: an int32 slot that holds it plus one (a fresh slot is
    zero: no token yet)."""

    @classmethod
    def tensors(cls, spec):
        out = super().tensors(spec)
        out["pairs"] = TensorSpec((spec["buckets"] + 1, spec["hidden"]))
        return out

    @classmethod
    def cache_need(cls, spec):
        return FixedState((1,), "int32")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.pairs = self.matrix(tensors["pairs"])
        self.rule = (int(spec["buckets"]), int(spec["mul_prev"]), int(spec["mul_cur"]))

    def forward(self, ctx, cache, out=None):
        return self.ops.embedding_pairs(ctx.token_ids, self.table, self.scale, self.pairs,
                                        rule=self.rule, ctx=ctx, view=cache, out=out)
