"""Host-side mirror of the reference's Python interface for the mapped-operator
path (reference package ``spherical_distortion`` = its ``layers/`` directory):
``nn.MappedConvolution``, ``nn.MappedTransposedConvolution``,
``nn.MappedMaxPool``, ``nn.Resample`` / ``nn.Unresample`` and the matching
``functional`` calls, with the reference's names, argument meaning and
assertion behaviour, on top of the drop-in ``_spherical_distortion_ext``.

The reference's own ``layers/nn`` and ``layers/functional`` files work unchanged
on top of ``_spherical_distortion_ext`` as well; this mirror exists so that the
path can be used and tested where the reference checkout is not installed.
"""
__version__ = "1.1.0"
