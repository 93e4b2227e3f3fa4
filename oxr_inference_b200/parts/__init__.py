"""Parts a decoder is assembled from; importing the package registers the built-in ones."""

from oxr_inference_b200.parts import attention, block, mlp, norm, rope  # noqa: F401  (register themselves)
from oxr_inference_b200.parts.base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                                           DeferredLinear, Embedding, FeedForward, GroupView, Head, LayerCache, Mixer, Norm, PagedKVNeed,
                                           ParamInfo, Part, PositionEncoding, Runtime, StateNeed, StepContext)
from oxr_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry



def __getattr__(name: str):
    # The decoder needs the cache's plan, and the cache needs this package's interfaces: import it on demand.
    if name == "DecoderModel":
        from oxr_inference_b200.parts.decoder import DecoderModel

        return DecoderModel
    raise AttributeError(name)


__all__ = [
    "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "DecoderModel", "DeferredLinear", "Embedding",
    "FeedForward", "GroupView", "Head", "LayerCache", "LayerSpec", "Mixer", "ModelSpec", "Norm", "PagedKVNeed", "ParamInfo", "Part", "PartSpec",
    "PositionEncoding", "Runtime", "ScheduleEntry", "StateNeed", "StepContext",
]
