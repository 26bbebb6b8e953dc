"""Enumerations shared with the native code (reference: ext_modules/include/layers/enum_export.h:8-29)."""
from ._C import (
    InterpolationType,
    DistortionType,
)  # noqa: F401
