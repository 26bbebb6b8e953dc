"""Same module name and functions as the reference's `_mapped_avg_pooling` (ext_modules/include/layers/mapped_avg_pooling_layer.h:89-94)."""
from ._C import mapped_avg_pool, mapped_avg_unpool  # noqa: F401
