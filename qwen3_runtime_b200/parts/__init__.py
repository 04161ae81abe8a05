# importing the modules registers the built-in parts
from . import (attention, block, conv_attention, embedding, experts, feed_forward, gated_memory,  # noqa: F401
               latent_attention, linear_state, norm, position, sink_attention, token_side)
from .base import (
    BuildContext,
    ParamSpec,
    Part,
    ResidualStream,
    StepContext,
    build_part,
    register_part,
    unregister_part,
)
from .model import DecoderModel

__all__ = [
    "BuildContext",
    "DecoderModel",
    "ParamSpec",
    "Part",
    "ResidualStream",
    "StepContext",
    "build_part",
    "register_part",
    "unregister_part",
]
