"""Build recipe for ``oracle/_ref/_C*.so`` -- the UNMODIFIED reference kernels of the hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this file or its output.

The reference sources are compiled where they lie (nothing is copied into this
repository); only the translation units the hot path needs are built, with the
reference's own optimisation level (``-O3``, ``fast_2d_gs/_C/setup.py:36-41``):

  src/pybind11.cpp                                  module entry / op registry
  src/gaussian_splatting/gs_2d_fast_preprocess.cu   preprocess + binning fwd/bwd
  src/gaussian_splatting/gs_2d_fast_redner.cu       compositing fwd/bwd
  src/gaussian_splatting/gaussian_prepare.cu        getHigherMsb (host helper the preprocess TU links to)
  src/other/cdist_top.cu                            top-1 neighbour (CUDA + CPU branch)
  src/other/adam_masked_update.cu                   masked Adam
  src/other/structural_similarity.cu                fused SSIM forward / backward

The reference passes ``-rdc=true`` without a device-link step, which makes the
stock extension un-importable; no TU above calls a device function of another
TU, so the flag is simply dropped here.

Besides the kernels, the reference's own Python packages (``fast_2d_gs``, ``utils``: ``*.py`` only) are copied to
``oracle/_ref/py`` (git-ignored like the rest of ``oracle/_ref``), so that the drop-in test can run the reference's
unmodified ``_Fast_Render`` / ``SparseGaussianAdam`` / ``utils.cdist_top`` over this library, and the benchmark its
PyTorch compositor, on a machine that has no reference checkout.

Usage:  python oracle/build_ref.py [--ref /path/to/reference] [--jobs N]
The output is used by the GPU parity tests (new CUDA == reference CUDA) and as
a timed baseline; it needs the reference checkout only at build time.
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
sys.path.insert(0, HERE)
from refpath import reference_root  # noqa: E402

UNITS = [
    "src/pybind11.cpp",
    "src/gaussian_splatting/gs_2d_fast_preprocess.cu",
    "src/gaussian_splatting/gs_2d_fast_redner.cu",
    "src/gaussian_splatting/gaussian_prepare.cu",
    "src/other/cdist_top.cu",
    "src/other/adam_masked_update.cu",
    "src/other/structural_similarity.cu",
]


def copy_python(ref_root):
    """``*.py`` of the reference's ``fast_2d_gs`` and ``utils`` packages -> oracle/_ref/py (unmodified)."""
    import shutil
    dst_root = os.path.join(OUT, "py")
    n = 0
    for pkg in ("fast_2d_gs", "utils"):
        for dirpath, _, files in os.walk(os.path.join(ref_root, pkg)):
            for f in files:
                if not f.endswith(".py"):
                    continue
                src = os.path.join(dirpath, f)
                dst = os.path.join(dst_root, os.path.relpath(src, ref_root))
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                if not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src):
                    shutil.copy2(src, dst)
                n += 1
    print(f"reference python: {n} files under {dst_root}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="reference checkout (default: $FSGS_REFERENCE_ROOT, else a "
                                                "directory named 'reference' beside this repository)")
    ap.add_argument("--jobs", type=int, default=4)
    args = ap.parse_args()
    ref_root = reference_root(args.ref)
    if ref_root is None:
        print("reference checkout not found; nothing built")
        return 0
    cdir = os.path.join(ref_root, "fast_2d_gs", "_C")
    os.makedirs(OUT, exist_ok=True)
    copy_python(ref_root)

    import pybind11
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    incs = [os.path.join(cdir, "include"), pybind11.get_include(), sysconfig.get_paths()["include"]]
    incs += ce.include_paths("cuda")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-O3", "-std=c++17", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-D__CUDA_NO_HALF_OPERATORS__"]
    common += [f"-I{p}" for p in incs]

    def compile_one(unit):
        src = os.path.join(cdir, unit)
        obj = os.path.join(OUT, os.path.basename(unit) + ".o")
        if os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src):
            return obj
        if unit.endswith(".cu"):
            cmd = ["nvcc", "-c", src, "-o", obj, "-gencode=arch=compute_100,code=sm_100", "--expt-relaxed-constexpr",
                   "-Xcompiler", "-fPIC", "-Wno-deprecated-declarations", "-w"] + common
        else:
            cmd = ["g++", "-c", src, "-o", obj, "-fPIC", "-Wno-deprecated-declarations", "-w"] + common
        print(" ".join(cmd[:6]), "...", flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(args.jobs) as ex:
        objs = list(ex.map(compile_one, UNITS))

    ext = sysconfig.get_config_var("EXT_SUFFIX")
    so = os.path.join(OUT, "_C" + ext)
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", so] + objs + [f"-L{p}" for p in libdirs] + \
           [f"-Wl,-rpath,{p}" for p in libdirs] + \
           ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    subprocess.check_call(link)
    print("built", so)
    return 0


if __name__ == "__main__":
    sys.exit(main())
