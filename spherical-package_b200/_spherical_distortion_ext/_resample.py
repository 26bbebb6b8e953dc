"""resample_to_map / resample_from_map (reference: ext_modules/include/layers/resample_layer.h:84-88)."""
from ._C import (
    resample_to_map,
    resample_from_map,
)  # noqa: F401
