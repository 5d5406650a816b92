"""Parts a layer is put together from.  Importing the package registers the built-in ones."""

from . import (  # noqa: F401
    attention, block, embedding, experts, gated_recurrence, latent_attention, linear_attention, matrix_memory, mlp, norm,
    parallel, rotary, streams,
)
from .base import (  # noqa: F401
    BLOCKS,
    EMBEDDINGS,
    HEADS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITIONS,
    KVNeed,
    ParamSpec,
    PendingSum,
    StateNeed,
    part_class,
    register_part,
)
