"""Parts a model is assembled from. Importing the package registers the built-in kinds."""
from .base import (BLOCKS, CONNECTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, CacheNeed, Embedding, FeedForward, Head,
                   Mixer, Norm, ParamDecl, Part, Runtime, register_block, register_embedding, register_feed_forward, register_head,
                   register_mixer, register_norm, register_position, register_connection, register_token_input, TOKEN_INPUTS, TokenInput)
from . import (attention, block, connections, gated_recurrence, latent_attention, mamba1, mamba2, matrix_memory, mlp, parallel, retention, sigmoid_attention, sink_attention, norms,  # noqa: F401
               positions, routed_mlp, token_input, vocab)  # noqa: F401  (registration)
from .linear import Linear

__all__ = ["BLOCKS", "CONNECTIONS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheNeed", "Embedding",
           "FeedForward", "Head", "Mixer", "Norm", "ParamDecl", "Part", "Runtime", "Linear", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm", "register_position", "register_connection",
           "register_token_input", "TOKEN_INPUTS", "TokenInput"]
