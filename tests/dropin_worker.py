"""Runs the reference's UNMODIFIED Python (``GS_2D_fast_render`` + backward, ``utils.cdist_top``,
``SparseGaussianAdam``) over one of two native operator modules and stores the results:

    python tests/dropin_worker.py fsgs out.npz     this library, through ``fsgs.install()``
    python tests/dropin_worker.py ref  out.npz     the reference's own compiled kernels (oracle/_ref/_C)

A process of its own per binding, because the reference reads its operators when its classes are defined.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "fast-sp-gs_b200"), os.path.join(ROOT, "oracle")):
    sys.path.insert(0, p)


def main(which, out_path):
    import refpy
    if which == "fsgs":
        import fsgs
        native = fsgs.install()
    else:
        sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
        import _C as native
    refpy.import_reference(native=native)
    from fast_2d_gs.renderer.gs_2d_fast_render import GS_2D_fast_render, _Fast_Render
    from fast_2d_gs.sparse_gaussian_adam import SparseGaussianAdam
    from utils.cdist_top import cdist_top
    assert _Fast_Render._preprocess_forward is native.gs_2d_fast_preprocess_forward
    assert SparseGaussianAdam._update_C is native.AdamMasksedUpdated

    from fsgs import workloads as wl
    P, W, H = 60_000, 640, 480
    s = wl.surfels(P, seed=31, log_scale_mean=-3.6, device="cuda")
    cam = wl.camera(W, H, eye=(0.4, -0.3, 4.0), device="cuda")
    names = ("means", "scales", "rots", "opac", "sh_dc", "sh_rest")
    leaves = [s[k].clone().requires_grad_() for k in names]
    groups = [dict(params=[p], lr=lr) for p, lr in zip(leaves, (1.6e-4, 5e-3, 1e-3, 0.05, 2.5e-3, 1.25e-4))]
    opt = SparseGaussianAdam(groups, lr=0.0, eps=1e-15)
    g = torch.Generator().manual_seed(32)
    ups = dict(images=torch.randn(3, H, W, generator=g).cuda(), opacity=torch.randn(H, W, generator=g).cuda(),
               normals=0.1 * torch.randn(3, H, W, generator=g).cuda(),
               distortion=0.1 * torch.randn(1, H, W, generator=g).cuda(),
               surf_depth=0.1 * torch.randn(1, H, W, generator=g).cuda())
    res = {}
    for step in range(3):
        means, scales, rots, opac, dc, rest = leaves
        out = GS_2D_fast_render(means, scales, rots, opac, (W, H), cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"],
                                sh_degree=3, sh_features=dc, sh_features_rest=rest)
        heads = [out[k] for k in ups]
        torch.autograd.backward(heads, [ups[k] for k in ups])
        if step == 0:
            for k in ("images", "opacity", "normals", "distortion", "surf_depth", "surf_normal", "radii"):
                res["out_" + k] = out[k].detach().cpu().numpy()
            for n, p in zip(names, leaves):
                res["grad_" + n] = p.grad.detach().cpu().numpy()
            res["grad_viewspace"] = out["viewspace_points"].grad.detach().cpu().numpy()
        opt.set_before_step(out["visibility_filter"], P)
        opt.step()
        opt.zero_grad(set_to_none=True)
    for n, p in zip(names, leaves):
        res["param_" + n] = p.detach().cpu().numpy()
    # the optimiser alone, on identical gradients: bit-exact
    q = torch.nn.Parameter(s["sh_rest"].clone())
    opt2 = SparseGaussianAdam([dict(params=[q], lr=1e-3)], lr=0.0, eps=1e-15)
    vis = (torch.rand(P, generator=g) < 0.7).cuda()
    for step in range(3):
        q.grad = torch.randn(q.shape, generator=g).cuda()
        opt2.set_before_step(vis, P)
        opt2.step()
    res["adam_param"] = q.detach().cpu().numpy()
    res["adam_exp_avg_sq"] = opt2.state[q]["exp_avg_sq"].cpu().numpy()
    # nearest / farthest control point through the reference's autograd wrapper
    x, c = wl.knn_points_c1(100_000, 512, 0)
    x, c = x.cuda().requires_grad_(), c.cuda().requires_grad_()
    d, i = cdist_top(x, c)
    d.sum().backward()
    res.update(cdist_dist=d.detach().cpu().numpy(), cdist_idx=i.cpu().numpy(), cdist_g1=x.grad.cpu().numpy(),
               cdist_g2=c.grad.cpu().numpy())
    d, i = cdist_top(x.detach(), c.detach(), True)
    res.update(cdist_far_dist=d.cpu().numpy(), cdist_far_idx=i.cpu().numpy())
    torch.cuda.synchronize()
    np.savez(out_path, **res)


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
