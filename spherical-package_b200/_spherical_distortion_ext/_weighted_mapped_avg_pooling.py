"""Same module name and functions as the reference's `_weighted_mapped_avg_pooling` (ext_modules/include/layers/weighted_mapped_avg_pooling_layer.h:109-114)."""
from ._C import weighted_mapped_avg_pool, weighted_mapped_avg_unpool  # noqa: F401
