from .base import Block, FeedForward, Mixer, Norm, PositionEncoding, Runtime
from .registry import build_part, register_part, registered_parts, unregister_part
from .spec import (AttentionSpec, BigramEmbeddingSpec, LatentAttentionSpec, LayerSpec, Mamba2Spec, MLSTMSpec, ModelSpec, MoESpec,
                   RMSNormSpec, RotarySpec, SwiGLUSpec)
from . import attention, block, embedding, latent_attention, mlp, moe, recurrent, rmsnorm, rotary   # registers the built-in parts
from .linear import Linear
