from .base import Block, FeedForward, Mixer, Norm, PositionEncoding, Runtime
from .registry import build_part, register_part, registered_parts, unregister_part
from .spec import AttentionSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec, SwiGLUSpec
from . import attention, block, mlp, rmsnorm, rotary   # registers the built-in parts
from .linear import Linear
