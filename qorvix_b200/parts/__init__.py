from .base import Block, FeedForward, Mixer, Norm, PositionEncoding, Runtime
from .registry import build_part, register_part, registered_parts, unregister_part
from .spec import (ActMLPSpec, AttentionSpec, BigramEmbeddingSpec, DiffAttentionSpec, LatentAttentionSpec, LayerSpec, LoopSpec, Mamba2Spec,
                   MLSTMSpec, ModelSpec, MoESpec, RMSNormSpec, RotarySpec, SwiGLUSpec, TableMoESpec, YarnScaling)
from . import (attention, block, diff_attention, embedding, latent_attention, loop, mlp, moe, recurrent, rmsnorm,   # registers the
               rotary)                                                                                              # built-in parts
from .linear import Linear
