"""Parts that layers are put together from: mixers, feed-forwards, norms, position encodings,
block arrangements, embedding and head.  Importing this package registers the built-in parts."""

from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
from .base import CallContext, KVCacheRequest, Part, StateRequest  # noqa: F401
from .registry import (build_part, lookup, register_block, register_embedding,  # noqa: F401
                       register_feed_forward, register_head, register_mixer, register_norm,
                       register_position)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec, WeightSpec  # noqa: F401
