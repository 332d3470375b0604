"""Imports the reference's own Python (unmodified) with a chosen native operator module behind it.

TEST INFRASTRUCTURE ONLY.  ``oracle/build_ref.py`` leaves a copy of the reference's ``fast_2d_gs`` and ``utils``
Python trees under ``oracle/_ref/py`` (git-ignored, like the compiled reference kernels beside it); this module puts
that copy -- or a live checkout -- on ``sys.path``, fabricates the third-party packages the reference imports but the
hot path never calls, and registers the native module the reference binds its operators to
(``fast_2d_gs/_C/__init__.py:15`` does ``from . import _C``).
"""
import importlib.abc
import importlib.machinery
import os
import sys
from unittest import mock

HERE = os.path.dirname(os.path.abspath(__file__))
REF_PY = os.path.join(HERE, "_ref", "py")

_ABSENT = ("matplotlib", "seaborn", "torchmetrics", "imageio", "lietorch", "plyfile", "pytorch3d", "pykdtree",
           "diff_surfel_rasterization", "diff_gaussian_rasterization", "dearpygui", "open3d", "trimesh", "lpips",
           "tensorboard", "tensorboardX", "skimage", "kornia", "roma", "pycolmap", "mediapy")


class _StubFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Answers imports of the packages above with MagicMock packages (none of them is reached on the hot path)."""

    def find_spec(self, name, path, target=None):
        if name.split(".")[0] in _ABSENT:
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = mock.MagicMock(name=spec.name)
        m.__path__ = []
        m.__name__ = spec.name
        m.__spec__ = spec
        m.__loader__ = self
        return m

    def exec_module(self, module):
        pass


def reference_python_root(explicit=None):
    """Directory to put on ``sys.path``: ``explicit``, else the copy under ``oracle/_ref/py``, else a live checkout
    (``refpath.reference_root``).  None when there is none."""
    from refpath import reference_root
    for c in (explicit, REF_PY, reference_root()):
        if c and os.path.isdir(os.path.join(c, "fast_2d_gs", "renderer")):
            return c
    return None


def import_reference(native=None, root=None):
    """Make ``fast_2d_gs`` / ``utils`` of the reference importable.  ``native``: the module object the reference's
    ``get_C_function`` should find as ``fast_2d_gs._C._C`` (this library's ``fsgs.install()`` result, or the compiled
    reference kernels ``oracle/_ref/_C``); None leaves the reference on its pure-PyTorch fallbacks.  Call before the
    first import of ``fast_2d_gs``: the reference reads its operators at class-definition time.  Returns the root."""
    root = reference_python_root(root)
    if root is None:
        raise ImportError("no reference Python found (run oracle/build_ref.py with a reference checkout present)")
    if "fast_2d_gs" in sys.modules:
        raise RuntimeError("fast_2d_gs is already imported; its operators were bound at class-definition time")
    if not any(isinstance(f, _StubFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, _StubFinder())
    if root not in sys.path:
        sys.path.insert(0, root)
    if native is not None:
        sys.modules["fast_2d_gs._C._C"] = native
    import warnings
    warnings.filterwarnings("ignore")
    return root
