"""Parts of a layer.  Importing this package registers the built-in ones."""

from tokensprint_b200.parts import attention, blocks, feed_forward, norms, position  # noqa: F401
from tokensprint_b200.parts.base import (  # noqa: F401
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    TRANSFORMS,
    Block,
    BuildContext,
    CacheNeed,
    FeedForward,
    GroupTables,
    LayerCache,
    Mixer,
    Norm,
    Part,
    PartSpec,
    PositionEncoding,
    StepContext,
    TensorSpec,
    Transform,
    build_part,
    register_part,
    unregister_part,
)
