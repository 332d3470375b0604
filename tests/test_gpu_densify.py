"""Densification on the device (clone / split selection, split children, move of parameters and Adam moments) against
the fixture produced by the reference's own ``densify`` and against the CPU oracle; statistics gathering; the scene
trains on afterwards.  Counts, order and copied rows exact; the children's positions and log-scales to 1e-6."""
import pytest
import torch

import densify_oracle as do
from util import load_golden

pytestmark = pytest.mark.gpu

NAMES = {"xyz": "_xyz", "sh_dc": "_features_dc", "sh_rest": "_features_rest", "scaling": "_scaling",
         "rotation": "_rotation", "opacity": "_opacity"}


def _scene_from(g, prefix="in"):
    from fsgs.scene import DynamicScene
    surf = dict(means=g[prefix + "_xyz"], log_scales=g[prefix + "_scaling"], rots_raw=g[prefix + "_rotation"],
                opac_raw=g[prefix + "_opacity"], sh_dc=g[prefix + "_features_dc"], sh_rest=g[prefix + "_features_rest"])
    return DynamicScene(surf, g[prefix + "_xyz"][:16].clone(), K=3, device="cuda")


def test_densify_matches_the_reference_fixture():
    g = load_golden("densify.npz", "cuda")
    scene = _scene_from(g)
    for name, a in NAMES.items():
        p = getattr(scene, name)
        scene.optimizer.state[p] = dict(step=torch.tensor(2.0), exp_avg=g["in_m" + a].clone(),
                                        exp_avg_sq=g["in_v" + a].clone())
    scene.enable_densification_stats()
    scene.grad_accum.copy_(g["accum"].reshape(-1))
    scene.grad_denom.copy_(g["denom"].reshape(-1))
    n_in, n_out = g["in_xyz"].shape[0], g["out_xyz"].shape[0]
    # the reference consumed the first rows of z, two columns of each
    flags_split = None
    n_clone, n_split = scene.densify(float(g["max_grad"]), float(g["extent"]), float(g["percent_dense"]), N=2,
                                     noise=g["z"][: 2 * (n_out - n_in), :2].contiguous()[: 2 * 10 ** 6])
    assert scene.num_points == n_out and n_clone + n_split == n_out - n_in
    for name, a in NAMES.items():
        p = getattr(scene, name).detach()
        ref = g["out" + a]
        n_old = n_out - 2 * n_split
        assert torch.equal(p[:n_old], ref[:n_old]), name            # kept originals and clones: copied rows
        if name in ("xyz", "scaling"):
            assert torch.allclose(p[n_old:], ref[n_old:], rtol=1e-6, atol=1e-6), name
        else:
            assert torch.equal(p[n_old:], ref[n_old:]), name
        st = scene.optimizer.state[getattr(scene, name)]
        assert torch.equal(st["exp_avg"], g["out_m" + a]) and torch.equal(st["exp_avg_sq"], g["out_v" + a]), name
        assert float(st["step"]) == 2.0
    assert scene.knn_idx.shape[0] == n_out and float(scene.grad_accum.abs().sum()) == 0.0


def test_densify_vs_oracle_and_training_goes_on():
    from fsgs import workloads as wl
    from fsgs.scene import DynamicScene, motion_at
    W, H, P = 160, 120, 6001
    surf = wl.surfels(P, seed=5, log_scale_mean=-3.0, log_scale_std=1.0)
    sp = wl.superpoints(surf["means"], M=64, seed=1)
    cam = {k: v.cuda() for k, v in wl.camera(W, H).items()}
    motion = motion_at(sp, sp["centres"], "cuda")
    gen = torch.Generator().manual_seed(9)
    g_img, g_op = torch.randn(3, H, W, generator=gen).cuda(), torch.randn(H, W, generator=gen).cuda()
    scene = DynamicScene(surf, sp["centres"], K=3, device="cuda")
    scene.enable_densification_stats()
    for _ in range(3):
        out = scene.train_step(cam, (W, H), motion, g_img, g_op)
    vis = out["visibility_filter"]
    # the parameters move between the steps, so a Gaussian may be visible in some of them only
    assert bool((scene.grad_denom[vis] > 0).all()) and float(scene.grad_denom.max()) == 3.0
    assert bool((scene.max_radii >= out["radii"].float()).all()) and bool((scene.max_radii[scene.grad_denom == 0] == 0).all())
    assert bool((scene.grad_accum[scene.grad_denom > 0] >= 0).all()) and float(scene.grad_accum.sum()) > 0
    thr = float(torch.quantile((scene.grad_accum / scene.grad_denom).nan_to_num(0.0), 0.8))
    names = ("xyz", "sh_dc", "sh_rest", "opacity", "scaling", "rotation")
    params = {n: getattr(scene, n).detach().cpu().clone() for n in names}
    moments = {n: (scene.optimizer.state[getattr(scene, n)]["exp_avg"].cpu().clone(),
                   scene.optimizer.state[getattr(scene, n)]["exp_avg_sq"].cpu().clone()) for n in names}
    z = torch.randn(2 * P, 2, generator=gen)
    ref, ref_m, n_clone_ref, n_split_ref = do.densify(params, moments, scene.grad_accum.cpu().clone(),
                                                      scene.grad_denom.cpu(), thr, 4.0, 0.01, z)
    n_clone, n_split = scene.densify(thr, 4.0, 0.01, noise=z[: 2 * n_split_ref].cuda())
    assert (n_clone, n_split) == (n_clone_ref, n_split_ref) and n_clone > 0 and n_split > 0
    for n in names:
        p = getattr(scene, n).detach().cpu()
        assert p.shape == ref[n].shape, n
        assert torch.allclose(p, ref[n], rtol=1e-6, atol=1e-6), n
        st = scene.optimizer.state[getattr(scene, n)]
        assert torch.equal(st["exp_avg"].cpu(), ref_m[n][0]) and torch.equal(st["exp_avg_sq"].cpu(), ref_m[n][1]), n
    out = scene.train_step(cam, (W, H), motion, g_img, g_op)   # the densified scene renders and steps
    assert out["radii"].shape[0] == scene.num_points and bool(torch.isfinite(out["images"]).all())
    assert float(scene.optimizer.state[scene.xyz]["step"]) == 4.0
    # prune keeps the statistics aligned
    remove = torch.rand(scene.num_points, generator=gen).cuda() < 0.3
    acc = scene.grad_accum.clone()
    scene.prune(remove)
    assert torch.equal(scene.grad_accum, acc[~remove])


def test_gather_rows_with_zero_rows():
    from fsgs import ops
    gen = torch.Generator().manual_seed(1)
    a = torch.randn(1000, 15, 3, generator=gen).cuda()
    b = torch.randint(0, 100, (1000, 3), generator=gen).cuda()           # int64 rows
    idx = torch.randint(-1, 1000, (2500,), generator=gen).to(torch.int32).cuda()
    oa, ob = ops.gather_rows([a, b], idx)
    sel = idx.long().clamp_min(0)
    za, zb = a[sel], b[sel]
    za[idx < 0] = 0
    zb[idx < 0] = 0
    assert torch.equal(oa, za) and torch.equal(ob, zb)
