from . import (attention, block, dense_mlp, feed_forward, general_attention, latent_attention, mixer_pair, norm,  # noqa: F401
               position, recurrent, routed_experts, state_space, token_input)  # noqa: F401  (register the built-in kinds)
from .base import (BuildContext, FixedStateNeed, PagedKVNeed, PagedLayerCache, Part, StateLayerCache, StepContext,
                   TensorSpec)
from .model import Model
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, TOKEN_INPUTS, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position, register_token_input)

__all__ = ["BuildContext", "FixedStateNeed", "PagedKVNeed", "PagedLayerCache", "Part", "StateLayerCache",
           "StepContext", "TensorSpec", "Model", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS",
           "TOKEN_INPUTS", "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "register_token_input"]
