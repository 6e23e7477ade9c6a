"""Parts a layer is put together from; importing this package registers the built-in ones."""
from .base import (  # noqa: F401
    Block, CacheNeed, DeferredNorm, DeltaPair, FeedForward, Mixer, Norm, Part, PositionEncoding, SequenceFilter, TensorDecl,
    build_part, plain_delta, register_part, registered,
)
from . import norm, rotary, attention, feed_forward, block, embedding  # noqa: F401
from . import short_conv, gated_norm, linear_recurrence, biased_attention, parallel, routed_experts  # noqa: F401,E402
from . import capped_attention, latent_attention  # noqa: F401,E402
from . import token_shift, sink_attention  # noqa: F401,E402
