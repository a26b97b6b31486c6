"""Parts a layer is assembled from.  Importing the package registers the built-in kinds."""
from . import (attention, block, channel_delta, decay_attention, differential_attention, embedding, feedforward,
               gated_attention, gated_linear_attention, grouped_routed, latent_attention, norm, parallel, rotary, routed,
               table_routed, transforms)  # noqa: F401  (registration)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, TRANSFORMS, Precision, Runtime,
                   register_arrangement, register_embedding, register_feed_forward, register_mixer, register_norm,
                   register_position, register_transform)

__all__ = ["ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "TRANSFORMS", "Precision",
           "Runtime", "register_arrangement", "register_embedding", "register_feed_forward", "register_mixer",
           "register_norm", "register_position", "register_transform"]
