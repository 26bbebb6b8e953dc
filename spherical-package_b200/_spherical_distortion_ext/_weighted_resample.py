"""Weighted resampling (reference: ext_modules/include/layers/weighted_resample_layer.h)."""
from ._C import (
    weighted_resample_to_map,
    weighted_resample_from_map,
)  # noqa: F401
