"""Same module name and functions as the reference's `_uv_resample` (ext_modules/include/layers/uv_resample_layer.h:103-108)."""
from ._C import resample_to_uv_maps, resample_from_uv_maps  # noqa: F401
