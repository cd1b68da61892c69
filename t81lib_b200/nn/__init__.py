"""``t81.nn`` counterpart: the ternary ``Linear`` layer."""

from .linear import Linear
from .sharded import ShardedLinear

__all__ = ["Linear", "ShardedLinear"]
