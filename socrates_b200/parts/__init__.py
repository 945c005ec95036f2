"""Parts a model is put together from: norm, position encoding, mixer, feed-forward,
their arrangement in a block, embedding and head.  Importing this package registers
the built-in kinds."""

from .base import (Branch, ParamSpec, Part, ResidualStream, build_part, register_part, registered,
                   unregister_part)
from . import norm, position, attention, feed_forward, block, embedding  # noqa: F401  (registration)
from .linear import Linear

__all__ = ["Branch", "ParamSpec", "Part", "ResidualStream", "build_part", "register_part",
           "registered", "unregister_part", "Linear"]
