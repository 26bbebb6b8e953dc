"""Argument checks shared by the functional calls (reference: layers/layer_utils.py:27-154)."""
from _spherical_distortion_ext._enums import DistortionType, InterpolationType  # noqa: F401


def _pair(v):
    return tuple(v) if hasattr(v, "__iter__") else (v, v)


def check_input_map_shape(input, sample_map):
    """Transposed / resample ops: the map has the input's spatial size (layer_utils.py:123-128)."""
    assert tuple(input.shape[2:4]) == tuple(sample_map.shape[0:2]), \
        "Input dimensions 2 and 3 must match sample map dimensions 0 and 1 ({} != {})".format(
            tuple(input.shape[2:4]), tuple(sample_map.shape[0:2]))


def check_args(input, sample_map, interp_weights, in_channels, kernel_size):
    """Same assertions, in the same order, as layer_utils.py:131-154."""
    has_kernel = kernel_size is not None
    weighted = interp_weights is not None
    assert input.dim() == 4, "Input must have 4 dimensions ({} != 4)".format(input.dim())
    want = 3 + int(has_kernel) + int(weighted)
    assert sample_map.dim() == want, "Sample map must have {} dimensions ({} != {})".format(want, sample_map.dim(), want)
    assert sample_map.shape[-1] == 2, \
        "Last dimension of sample map must have size 2 ({} != 2)".format(sample_map.shape[-1])
    if weighted:
        assert interp_weights.dim() == want - 1, \
            "Interpolation weights must have {} dimensions ({} != {})".format(want - 1, interp_weights.dim(), want - 1)
    assert input.dtype == sample_map.dtype, \
        "Input and sample map must be the same dtype ({} != {})".format(input.dtype, sample_map.dtype)
    if weighted:
        assert input.dtype == interp_weights.dtype, \
            "Input and interpolation weights must be the same dtype ({} != {})".format(input.dtype, interp_weights.dtype)
    if in_channels is not None:
        assert input.shape[1] == in_channels, \
            "Number of input channels must match weight parameter ({} != {})".format(input.shape[1], in_channels)
    if has_kernel:
        assert sample_map.shape[2] == kernel_size, \
            "Kernel size of sample map must match weight parameter ({} != {})".format(sample_map.shape[2], kernel_size)
    if weighted:
        assert sample_map.shape[-2] == interp_weights.shape[-1], \
            "Sample map and interpolation weights should have the same number of interpolation points " \
            "({} != {})".format(sample_map.shape[-2], interp_weights.shape[-1])
