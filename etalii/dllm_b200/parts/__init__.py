from . import (attention, block, differential_attention, embedding, feed_forward, latent_attention,  # noqa: F401
               linear_attention, mixture, norm, parallel, position, reentry, short_conv, sigmoid_attention,
               token_input)  # (register the built-in parts)
from .registry import build_part, part_factory, register_part, unregister_part  # noqa: F401
from .spec import LayerSpec, ModelSpec, ParamSpec, PartSpec, ScheduleEntry  # noqa: F401
