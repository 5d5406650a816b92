"""Parts a layer is put together from.  Importing the package registers the built-in ones."""

from . import attention, block, embedding, experts, latent_attention, linear_attention, matrix_memory, mlp, norm, parallel, rotary  # noqa: F401
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
