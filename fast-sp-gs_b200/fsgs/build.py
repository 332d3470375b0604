"""Builds ``libfsgs.so`` (sm_100a) next to the sources.  ``python -m fsgs.build`` or ``fsgs.build.build()``."""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(PKG), "csrc")
LIB = os.path.join(os.path.dirname(PKG), "lib", "libfsgs.so")
SOURCES = ["fsgs_preprocess.cu", "fsgs_bin.cu", "fsgs_blend.cu", "fsgs_knn.cu", "fsgs_epilogue.cu", "fsgs_loss.cu", "fsgs_compact.cu", "fsgs_step.cu", "fsgs_motion.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-extended-lambda", "-Xcompiler", "-fPIC"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(os.path.dirname(PKG)), "include", "fsgs.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source for sm_100a and link the shared library.  Returns the library path."""
    if not force and not _stale():
        return LIB
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    objs, procs = [], []
    for src in SOURCES:
        obj = os.path.join(os.path.dirname(LIB), src + ".o")
        cmd = ["nvcc", "-c", os.path.join(CSRC, src), "-o", obj] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    subprocess.check_call(["nvcc", "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                                  "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
