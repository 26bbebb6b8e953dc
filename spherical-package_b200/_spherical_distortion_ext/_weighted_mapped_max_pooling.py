"""Weighted mapped max pooling (reference: ext_modules/include/layers/weighted_mapped_max_pooling_layer.h)."""
from ._C import (
    weighted_mapped_max_pool,
    weighted_mapped_max_unpool,
)  # noqa: F401
