"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""

from .base import (  # noqa: F401
    Block,
    FeedForward,
    Mixer,
    Norm,
    PagedKVSpec,
    Part,
    PartSpec,
    PositionEncoding,
    StateSpec,
    TensorSpec,
    build_part,
    register_part,
)
from . import attention, block, feed_forward, norm, rotary  # noqa: F401,E402
