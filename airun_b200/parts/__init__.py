"""Parts of a model; importing the package registers the built-in ones."""
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, PagedKVSpec, StateSpec, NormedActivations,
                   ResidualSink,
                   register_part, make_part, registered_parts)
from . import norm, rope, attention, mlp, block, embedding  # noqa: F401  (registration)
