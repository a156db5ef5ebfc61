"""Makes the reference's import paths resolve to this package (``install_as_swin3d``: the Python
level, this package's Functions replace the reference's) or to this package's re-creation of its two
compiled modules (``install_pybind_modules``: the pybind level, the reference's Python stays).

``Swin3D/modules/swin3d_layers.py:16-24`` imports ``Swin3D.sparse_dl.attn.attn_coff`` and
``Swin3D.sparse_dl.knn``.  ``install_as_swin3d()`` registers this package's modules under those
names so that the reference's ``WindowAttention``, ``GridKNNDownsample`` and ``Upsample`` call the
kernels of libswin3d_b200.so without a change to their source.
"""
import importlib
import sys
import types


def install_pybind_modules(force: bool = False) -> None:
    """The other level of the boundary: keeps the reference's own ``Swin3D/sparse_dl/attn/attn_coff.py``
    and ``Swin3D/sparse_dl/knn/knn.py`` byte for byte and only supplies the two compiled modules they
    import, ``Swin3D.sparse_dl.attn_cuda`` (Swin3D/src/attn/attn_api.cpp:20-24) and
    ``Swin3D.sparse_dl.knn_cuda`` (Swin3D/src/knn/knn_api.cpp:4-6), implemented over libswin3d_b200.so.
    Call before ``import Swin3D.sparse_dl`` (the reference package must be importable)."""
    for alias, target in (("Swin3D.sparse_dl.attn_cuda", "swin3d_b200.sparse_dl.attn_cuda"),
                          ("Swin3D.sparse_dl.knn_cuda", "swin3d_b200.sparse_dl.knn_cuda")):
        if alias in sys.modules and not force:
            continue
        sys.modules[alias] = importlib.import_module(target)


def install_as_swin3d(force: bool = False) -> None:
    """Call before ``import Swin3D.modules`` / ``Swin3D.models``."""
    mapping = {
        "Swin3D.sparse_dl": "swin3d_b200.sparse_dl",
        "Swin3D.sparse_dl.attn": "swin3d_b200.sparse_dl.attn",
        "Swin3D.sparse_dl.attn.attn_coff": "swin3d_b200.sparse_dl.attn.attn_coff",
        "Swin3D.sparse_dl.knn": "swin3d_b200.sparse_dl.knn",
        "Swin3D.sparse_dl.knn.knn": "swin3d_b200.sparse_dl.knn.knn",
    }
    if "Swin3D" not in sys.modules:
        try:
            importlib.import_module("Swin3D")
        except ImportError:
            pkg = types.ModuleType("Swin3D")
            pkg.__path__ = []
            sys.modules["Swin3D"] = pkg
    for alias, target in mapping.items():
        if alias in sys.modules and not force:
            continue
        mod = importlib.import_module(target)
        sys.modules[alias] = mod
        parent, _, leaf = alias.rpartition(".")
        if parent in sys.modules:
            setattr(sys.modules[parent], leaf, mod)


def patch_basic_layer(basic_layer_cls) -> None:
    """Replaces ``BasicLayer.get_index01`` (Swin3D/modules/swin3d_layers.py:789-822) of the given
    class by the window builder of this package, so that the two index constructions per stage
    (:858-859) no longer enumerate window cells through MinkowskiEngine pooling.  The method keeps
    its signature ``(self, sp, local_xyz, colors)`` and reads ``self.window_size``; the shifted
    sparse tensor the caller passes for the odd blocks is grouped by its (already shifted)
    coordinates."""
    from . import window

    def get_index01(self, sp, local_xyz, colors):
        return window.get_index01(sp, local_xyz, colors, self.window_size)

    basic_layer_cls.get_index01 = get_index01
