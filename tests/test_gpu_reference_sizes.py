"""The whole operator chain against the reference's own CUDA kernels (oracle/_ref) at the sizes of the benchmark
configurations: 300 000 surfels at 800x800, one view of the 500 000-surfel 1352x1014 batch, and the binning of the
2 M-surfel 1920x1080 configuration.

Bars: per-Gaussian preprocess outputs and tile lists bit-equal; images (colour, opacity and all eight auxiliary
channels) within 1e-4 max abs; n_contrib equal; gradients within 1e-3 relative L2 per tensor.
"""
import pytest
import torch

from util import assert_preprocess_equal, reference_ext, rel_l2

pytestmark = pytest.mark.gpu

IMG_TOL = 1e-4
GRAD_TOL = 1e-3
EXTRAS = ["depth", "normal.x", "normal.y", "normal.z", "median depth", "distortion", "M1", "M2"]


@pytest.fixture(scope="module")
def ref():
    r = reference_ext()
    if r is None:
        pytest.skip("oracle/_ref not built")
    return r


def _scene(name, view):
    from fsgs import workloads as wl
    cfg = wl.CONFIGS[name]
    s = wl.surfels(cfg["P"], seed=0, log_scale_mean=cfg["log_scale_mean"], log_scale_std=cfg["log_scale_std"],
                   device="cuda")
    eye = wl.arc_eye(cfg["radius"], view, cfg["views"]) if "views" in cfg else (0.0, 0.0, 4.0)
    return cfg, s, wl.camera(cfg["W"], cfg["H"], eye=eye, device="cuda")


def _pre_args(cfg, s, cam):
    return (cfg["W"], cfg["H"], 3, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"], s["sh_rest"],
            cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"], None, None, None)


@pytest.mark.parametrize("name,view", [("train_300k_800", 0), ("multiview_500k_1352x1014", 3),
                                       ("multiview_500k_1352x1014", 12)])
def test_chain_vs_reference_cuda(ref, name, view):
    from fsgs import ops
    cfg, s, cam = _scene(name, view)
    P, W, H = cfg["P"], cfg["W"], cfg["H"]
    mine = ops.gs_2d_fast_preprocess_forward(*_pre_args(cfg, s, cam), True)
    theirs = ref.gs_2d_fast_preprocess_forward(*_pre_args(cfg, s, cam), False)
    torch.cuda.synchronize()
    assert_preprocess_equal(mine, theirs)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = mine

    # compositing forward on identical inputs
    fa = ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity, trans_mat, inverse_m,
                                       point_list, ranges, None, None, None, None, None)
    fb = ref.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity, trans_mat, inverse_m,
                                       point_list, ranges, None, None, None, None, None)
    torch.cuda.synchronize()
    assert float((fa[0] - fb[0]).abs().max()) < IMG_TOL, "colour"
    assert float((fa[1] - fb[1]).abs().max()) < IMG_TOL, "opacity"
    for ch, label in enumerate(EXTRAS):
        assert float((fa[2][ch] - fb[2][ch]).abs().max()) < IMG_TOL, label
    assert torch.equal(fa[4], fb[4])

    # compositing backward, upstream gradients on colour, opacity, depth, normals, median depth and distortion
    g = torch.Generator().manual_seed(23)
    g_img, g_op = torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()
    g_ext = torch.zeros(8, H, W, device="cuda")
    g_ext[:6] = torch.randn(6, H, W, generator=g).cuda() * 0.1
    ga = ops.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, None, fa[0], fa[1],
                                        fa[2], None, g_img, g_op, g_ext, None, ranges, point_list, fa[4], 0.2, 100.0,
                                        None, None, None, None, None, None)
    gb = ref.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, None, fb[0], fb[1],
                                        fb[2], None, g_img, g_op, g_ext, None, ranges, point_list, fb[4], 0.2, 100.0,
                                        None, None, None, None, None, None)
    torch.cuda.synchronize()
    names = ["colors", "means2D", "trans_mat", "inverse_m", "normal_opacity"]
    for label, x, y in zip(names, ga, gb):
        assert rel_l2(x, y) < GRAD_TOL, f"{label}: {rel_l2(x, y)}"

    # preprocess backward on identical upstream gradients (the reference's, so that only this stage differs)
    def run(mod, grads):
        gm, gs, gr, go = (torch.zeros(P, k, device="cuda") for k in (3, 2, 4, 1))
        gsh, grest = torch.zeros_like(s["sh_dc"]), torch.zeros_like(s["sh_rest"])
        gm2d = grads[1].clone()
        mod.gs_2d_fast_preprocess_backward(W, H, 3, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                           s["sh_rest"], cam["Tw2v"], cam["Tv2s"], cam["campos"], trans_mat, radii,
                                           colors, normal_opacity, gm2d, grads[2], grads[3], None, grads[0], grads[4],
                                           gm, gs, gr, go, gsh, grest, None, None)
        return gm, gs, gr, go, gsh, grest, gm2d

    pa, pb = run(ops, gb), run(ref, gb)
    torch.cuda.synchronize()
    for label, x, y in zip(["means", "scales", "rots", "opacity", "sh_dc", "sh_rest", "means2D proxy"], pa, pb):
        assert rel_l2(x, y) < GRAD_TOL, f"{label}: {rel_l2(x, y)}"


def test_stress_lists_vs_reference_cuda(ref):
    """2 M surfels at 1920x1080: per-Gaussian outputs and tile lists equal the reference kernels'."""
    from fsgs import ops
    cfg, s, cam = _scene("stress_2m_1080p", 7)
    mine = ops.gs_2d_fast_preprocess_forward(*_pre_args(cfg, s, cam), True)
    theirs = ref.gs_2d_fast_preprocess_forward(*_pre_args(cfg, s, cam), False)
    torch.cuda.synchronize()
    assert_preprocess_equal(mine, theirs)
