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


def pair_keys(ranges, point_list):
    """(tile << 32 | Gaussian) of every listed pair, in list order."""
    lens = ranges[:, 1] - ranges[:, 0]
    tile = torch.repeat_interleave(torch.arange(ranges.shape[0], device=ranges.device), lens)
    return tile * (1 << 32) + point_list[: int(lens.sum())].long()


def assert_preprocess_equal(mine, theirs):
    """Outputs of gs_2d_fast_preprocess_forward against the reference kernels': everything bit-equal (colours to
    2e-6: the SH polynomial is not pinned operation by operation), tile lists included."""
    names = ["means2D", "colors", "trans_mat", "inverse_m", "normal_opacity", "depths", "radii"]
    for n, a, b in zip(names, mine, theirs):
        assert a.shape == b.shape, n
        if n == "colors":
            assert float((a - b).abs().max()) < 2e-6, n
        else:
            assert torch.equal(a, b), f"{n}: {(a != b).sum().item()} of {a.numel()} elements differ"
    assert mine[8].shape == theirs[8].shape  # numel == sum of rectangle areas
    if not (torch.equal(mine[7], theirs[7]) and torch.equal(mine[8], theirs[8])):
        a, b = pair_keys(mine[7], mine[8]), pair_keys(theirs[7], theirs[8])
        _, cnt = torch.unique(torch.cat([a, b]), return_counts=True)
        raise AssertionError(f"tile lists differ: {int((cnt == 1).sum())} of {b.numel()} pairs are in one list only")
