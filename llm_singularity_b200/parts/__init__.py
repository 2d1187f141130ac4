"""Parts a model is assembled from: norms, position encodings, mixers,
feed-forwards and block arrangements, each chosen by the ``kind`` of its spec."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheSpec, CompositeCacheSpec, KVCacheView, LatentCacheView,
                   LatentPagesSpec, PagedKVSpec, ParamSpec, Part, Runtime, StateSpec, StateView, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position)
from . import (attention, block, delta, embedding, kv_attention, latent, memory, mlp, moe, norm, parallel, recurrence,  # noqa: F401
               rglru, rotary)                                                                            # (registration)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "CacheSpec", "CompositeCacheSpec", "KVCacheView", "LatentCacheView",
           "LatentPagesSpec", "PagedKVSpec", "ParamSpec", "Part", "Runtime", "StateSpec", "StateView", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position"]
