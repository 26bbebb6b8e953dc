"""Helpers for running the reference's unmodified Python layer (`layers/`, installed as `spherical_distortion`) on
top of this package.

The reference's `spherical_distortion.util` imports a few third-party packages at import time that have nothing to
do with the mapped operators (image and mesh file IO, plotting: layers/util/io.py:1-6,
layers/util/distortion.py:2).  Where they are not installed, `install_placeholders()` registers empty stand-in
modules under their names so that the import chain completes; anything that would really need them fails when it is
used, not when the package is imported.  Modules that are installed are left alone."""
import importlib.util
import sys
import types

THIRD_PARTY = ("skimage", "skimage.io", "matplotlib", "matplotlib.pyplot", "matplotlib.patches", "plyfile", "OpenEXR",
               "Imath", "visdom")


def _missing(name):
    if name in sys.modules:
        return False
    try:
        return importlib.util.find_spec(name) is None
    except (ImportError, ValueError, AttributeError):
        return True


def install_placeholders(names=THIRD_PARTY):
    """Register stand-ins for the third-party modules in `names` that cannot be imported; returns their names."""
    made = []
    for name in names:
        if not _missing(name):
            continue
        mod = types.ModuleType(name)
        mod.__doc__ = "placeholder registered by _spherical_distortion_ext.reference_compat (package not installed)"
        mod.__path__ = []
        sys.modules[name] = mod
        parent, _, child = name.rpartition(".")
        if parent and parent in sys.modules:
            setattr(sys.modules[parent], child, mod)
        made.append(name)
    return made


def mount_reference_layers(layers_dir):
    """Make `import spherical_distortion` resolve to the reference's own `layers/` folder (what its setup.py installs
    under that name, setup.py:211-228), without copying it."""
    import importlib.machinery
    import os
    init = os.path.join(layers_dir, "__init__.py")
    if not os.path.exists(init):
        raise FileNotFoundError(init)
    spec = importlib.machinery.ModuleSpec("spherical_distortion", importlib.machinery.SourceFileLoader(
        "spherical_distortion", init), origin=init, is_package=True)
    spec.submodule_search_locations = [layers_dir]
    mod = importlib.util.module_from_spec(spec)
    sys.modules["spherical_distortion"] = mod
    spec.loader.exec_module(mod)
    return mod
