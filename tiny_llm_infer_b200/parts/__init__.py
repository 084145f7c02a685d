"""Parts of a layer: mixers, feed-forwards, norms, position encodings and block
arrangements, each with its sizes and constants as parameters and none aware of the
model it is used in.  Importing this package registers the built-in parts."""
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, lookup, register,
                       unregister)
from .spec import (CacheSpec, ExecEntry, LayerSpec, ModelDescription, ParamSpec, PartSpec,
                   StateSpec)
