"""Import-time stand-in for the reference's `_mesh` module (CGAL triangle meshes, icospheres, tangent-plane
intersection: ext_modules/src/cpp/triangle_mesh.cpp).  Mesh utilities are outside the mapped-operator path this
package rebuilds; the reference's Python layer imports `_mesh` unconditionally
(layers/util/icosahedron_functions.py:5, layers/util/tangent_images.py:11), so the name must resolve for
`import spherical_distortion` to succeed.  Every attribute resolves to an object that raises on use."""


class _Unavailable:
    def __init__(self, name):
        self._name = name

    def _fail(self, *a, **kw):
        raise ImportError("_spherical_distortion_ext._mesh.%s is not provided by the B200 mapped-operator package: "
                          "build the reference's own `_mesh` extension (it needs CGAL) for mesh utilities" % self._name)

    __call__ = _fail

    def __getattr__(self, item):
        if item.startswith("__"):
            raise AttributeError(item)
        return _Unavailable(self._name + "." + item)


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    return _Unavailable(name)
