"""Mapped max pooling (reference: ext_modules/include/layers/mapped_max_pooling_layer.h:92-97)."""
from ._C import (
    mapped_max_pool,
    mapped_max_unpool,
)  # noqa: F401
