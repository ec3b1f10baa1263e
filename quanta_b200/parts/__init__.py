"""Parts a model is put together from; importing this package registers the built-in ones."""
from . import attention, block, conv, delta_rule, dense, gated_delta, gla, latent_attention, moe, norms, rotary, state_space, window_attention  # noqa: F401
from .base import (Addends, Block, CacheSpec, CacheStream, Embedding, FeedForward, Head, KeepAll, KVCacheSpec,  # noqa: F401
                   LayerCache, Mixer, Norm, NormedPending, Part, StreamsPending, PositionEncoding, Retention, StepContext, TensorSpec, TimeConv, Window, WindowAndOpenBlock, make,
                   register, registered)
from .spec import ModelSpec, ScheduleEntry  # noqa: F401
