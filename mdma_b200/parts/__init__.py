"""Parts a layer is put together from; importing this package registers them."""
from . import (attention, block, distance_attention, embedding, gating, latent_attention, linear_attention, mlp, norm, recurrent,  # noqa: F401
               rotary, routed_mlp, talking_attention)
from .base import Part, Runtime
from .linear import Linear

__all__ = ["Part", "Runtime", "Linear"]
