"""Drop-in installation: present the operators as the reference's compiled extension.

The reference resolves its native functions by name from the module ``fast_2d_gs._C._C`` at class-definition
time (``fast_2d_gs/_C/__init__.py:15,41-42``; ``renderer/gs_2d_fast_render.py:24-25,593-596``;
``utils/cdist_top.py:42-44``; ``sparse_gaussian_adam.py:11``).  ``install()`` registers a module of that name
holding this library's operators; call it BEFORE the first ``import fast_2d_gs`` / ``import utils``.
Operators this library does not provide resolve to ``None`` exactly as with an extension built without them.
"""
import sys
import types


def install(module_name="fast_2d_gs._C._C"):
    from .ops import REFERENCE_OPS
    from ._lib import lib
    lib()  # fail now, loudly, if libfsgs.so is missing
    mod = sys.modules.get(module_name)
    if mod is None:
        mod = types.ModuleType(module_name)
        mod.__doc__ = "fsgs operators (B200) standing in for the Fast-SP-GS CUDA extension"
        sys.modules[module_name] = mod
    for name, op in REFERENCE_OPS.items():
        setattr(mod, name, op)
    return mod
