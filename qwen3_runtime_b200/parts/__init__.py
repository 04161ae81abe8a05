# importing the modules registers the built-in parts
from . import (attention, block, conv_attention, differential_attention, embedding, experts,  # noqa: F401
               feed_forward, gated_memory, latent_attention, linear_state, norm, position, sink_attention, token_side)
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
