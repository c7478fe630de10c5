from .spec import PartSpec, BlockSpec, ModelSpec, RunStep
from .base import (Runtime, CacheNeed, PagedKV, PagedKVView, PagedLatent, PagedLatentView, GatedSum, SlotState, SlotStateView, HostBatch, Plan, ScaledSum, Part, Mixer,
                   FeedForward, Norm, PositionEncoding, Embedding)
from .registry import (register_mixer, register_feed_forward, register_norm, register_position_encoding,
                       register_block, register_embedding, register_architecture, architecture, architectures)
from . import (norm, rope, attention, capped_attention, recurrent, mlp, block, normed_attention, latent_attention,
               experts, embedding)  # registers the parts that ship with the engine
from .block import Block
