"""Same module name and functions as the reference's `_voting_resample` (ext_modules/include/layers/voting_resample_layer.h:60-63)."""
from ._C import voting_resample_to_map  # noqa: F401
