from .base import FAMILIES, Part, WeightSpec, build_part, part_class, register_part, registered_parts
from .stream import ResidualStream
from . import block, feed_forward, io, mixer, norm, position  # noqa: F401  (registers the built-in parts)

__all__ = ["FAMILIES", "Part", "WeightSpec", "build_part", "part_class", "register_part", "registered_parts",
           "ResidualStream"]
