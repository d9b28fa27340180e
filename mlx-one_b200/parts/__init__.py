from . import blocks, embeddings, feed_forwards, mixers, norms, positions  # register the built-in kinds
from .base import (Block, Embedding, FeedForward, FixedState, Mixer, Norm, NormedInput, PagedKeyValues, PagedView,
                   Part, PositionEncoding, Runtime, StateView, StepContext)
from .model import Model, cache_entries, expected_tensors
from .registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from .spec import Injection, LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec

__all__ = ["Block", "Embedding", "FeedForward", "FixedState", "Mixer", "Norm", "NormedInput", "PagedKeyValues",
           "PagedView", "Part", "PositionEncoding", "Runtime", "StateView", "StepContext",
           "Model", "cache_entries", "expected_tensors", "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "MIXERS",
           "NORMS", "POSITIONS", "Injection", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec",
           "TensorSpec"]
