from . import (attention, connector, dyt, embedding, gated_delta, hgrn2, latent_attention, layernorm, moe, parallel,  # noqa: F401
               polynorm, residual_gate, retention, rmsnorm, rope, shifted, shortconv, swiglu, timemix, token_side)      # (registers the parts)
from .base import (CONNECTORS, Connector, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Embedding,
                   FeedForward, FixedState, Head, Mixer, Norm, PagedKV, ParamDecl, Part, PositionEncoding, ResidualGate, Shared,
                   SideInput,
                   build_part, register_part)
from .spec import LayerSpec, ModelSpec, PartSpec, Run
