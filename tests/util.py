"""Shared helpers of the test-suite."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def load_golden(name, device="cpu"):
    z = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(z[k]).to(device) for k in z.files}


def rel_l2(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def reference_ext():
    """The reference's own CUDA kernels (built by oracle/build_ref.py), or None when not built."""
    d = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(d) or not any(f.startswith("_C") and f.endswith(".so") for f in os.listdir(d)):
        return None
    if d not in sys.path:
        sys.path.insert(0, d)
    try:
        import _C as ref
        return ref
    except ImportError:
        return None


def make_scene(P, W, H, seed=0, log_scale_mean=-3.0, eye=(0.3, -0.4, 4.0), device="cuda"):
    from fsgs import workloads as wl
    s = wl.surfels(P, seed=seed, log_scale_mean=log_scale_mean, device=device)
    cam = wl.camera(W, H, eye=eye, device=device)
    return s, cam


def cpu(t):
    return None if t is None else t.detach().cpu()
