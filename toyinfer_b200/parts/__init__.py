"""Model parts; importing the package registers the implementations it ships."""
from .base import (
    Block,
    BuildContext,
    Embedding,
    FeedForward,
    Head,
    KVRequest,
    Mixer,
    Norm,
    ParamSpec,
    Part,
    PartSpec,
    PositionEncoding,
    StateRequest,
    build_part,
    register_part,
    registered_parts,
    unregister_part,
)
from . import (norms, rope, attention, latent_attention, lightning, mlp, block, parallel_block, ends,  # noqa: F401  (registration)
               hyper_block, rglru, biased_attention, channel_delta, sandwich_block, window_attention, mamba2, side_by_side)
from .model import DecoderModel, LayerSpec, ModelSpec, ScheduleEntry

__all__ = [
    "Block", "BuildContext", "Embedding", "FeedForward", "Head", "KVRequest", "Mixer", "Norm", "ParamSpec", "Part",
    "PartSpec", "PositionEncoding", "StateRequest", "build_part", "register_part",
    "registered_parts", "unregister_part", "DecoderModel", "LayerSpec", "ModelSpec", "ScheduleEntry",
]
