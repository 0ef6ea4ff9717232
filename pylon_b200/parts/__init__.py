"""Parts a layer is put together from.  Importing the package registers the built-in kinds."""
from pylon_b200.parts import attention, block, mlp, norm, rope  # noqa: F401  (registration)
from pylon_b200.parts.base import (  # noqa: F401
    BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheNeed, FeedForward, KVNeed, LayerCache,
    Mixer, Norm, Part, PositionEncoding, ResidualStream, StateNeed, StepView, TensorDecl,
)
from pylon_b200.parts.spec import LayerSpec, ModelSpec, PartSpec  # noqa: F401
