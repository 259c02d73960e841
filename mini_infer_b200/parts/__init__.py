"""Parts a decoder is put together from (see ``base`` for the interfaces)."""

from .base import (  # noqa: F401
    Arrangement,
    DeferredNorm,
    FeedForward,
    GroupView,
    KVNeed,
    LayerCache,
    Mixer,
    Norm,
    ParamDecl,
    Part,
    PlanNeeds,
    Position,
    StateNeed,
    StepContext,
    StreamSink,
    build_part,
    lookup,
    register_arrangement,
    register_embedding,
    register_feed_forward,
    register_head,
    register_mixer,
    register_norm,
    register_position,
)
from .model import DecoderModel  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
