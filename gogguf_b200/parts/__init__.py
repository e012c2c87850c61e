"""Parts a model is put together from.  Importing this package registers the built-in kinds."""
from . import registry
from .base import Linear, Runtime, StepContext, Workspace
from . import (norm, position, attention, latent_attention, retention, recurrence, side_by_side, input_conv, feedforward,  # noqa: F401
               experts, gates, block, embedding, stream, token_shift, diff_attention, linear_recurrent)      # (registration)
from .registry import (register_arrangement, register_embedding, register_feed_forward, register_head,
                       register_gate, register_mixer, register_norm, register_position, register_stream)
