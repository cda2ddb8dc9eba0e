"""The parts a model is put together from.  Importing this package registers the built-in
parts under their names."""
from . import (attention, block, delta_rule, depth_mix, embedding, gated_scan, head, hyper, latent_attention, mlp,  # noqa: F401
               mlstm, norm, position, retention, routed, selective_scan)  # (registration)
from .base import (CONNECTORS, DEPTH_MIXES, FEED_FORWARDS, HEADS, EMBEDDINGS, MIXERS, NORMS, POSITIONS, Connector, DepthMix, Embedding, FeedForward, Head,
                   KVCacheSpec, KVCacheView, Mixer, Norm, ParamSpec, Part, PositionEncoding, StateSpec,
                   StepContext, TensorRef, Workspace, register_connector, register_depth_mix, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position)
from .block import BLOCKS, Block, register_block

__all__ = [n for n in dir() if not n.startswith("_")]
