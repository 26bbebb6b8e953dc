"""Drop-in replacement for the reference's native package of the same name
(its modules are built by the reference's setup.py:62-210), for the
mapped-operator path only, backed by hand-written sm_100a CUDA.

The compiled host extension ``_C`` (csrc/torch_shim.cpp) calls the C ABI of
``libsphmap.so`` (include/sphmap.h).  Both are built in-tree by build.py /
setup.py.  Importing this package without them fails loudly: there is no CPU
or pure-PyTorch fallback.
"""
import os as _os

_here = _os.path.dirname(_os.path.abspath(__file__))
if not _os.path.exists(_os.path.join(_here, "libsphmap.so")):
    raise ImportError("libsphmap.so has not been built: run `python build.py` in " + _os.path.dirname(_here))

import torch as _torch  # noqa: E402,F401  (libtorch must be loaded before the extension)

from . import _C  # noqa: E402

set_precision = _C.set_precision
get_precision = _C.get_precision
clear_plan_cache = _C.clear_plan_cache
plan_cache_size = _C.plan_cache_size
device_status = _C.device_status
set_companions = _C.set_companions
clear_companions = _C.clear_companions
