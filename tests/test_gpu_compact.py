"""GPU tests of the row compaction used for pruning (all tensors and optimiser moments in one gather)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,p", [(1, 1.0), (1, 0.0), (1023, 0.5), (1025, 0.9), (4096, 0.0), (300_000, 0.7),
                                 (2_000_000, 0.31)])
def test_compact_rows_equals_boolean_indexing(N, p):
    from fsgs import ops
    g = torch.Generator(device="cuda").manual_seed(N)
    keep = torch.rand(N, device="cuda", generator=g) < p
    ts = [torch.randn(N, 3, device="cuda", generator=g), torch.randn(N, 15, 3, device="cuda", generator=g),
          torch.randn(N, 1, device="cuda", generator=g), torch.randn(N, device="cuda", generator=g),
          torch.randint(0, 1 << 40, (N, 3), device="cuda", generator=g),
          torch.randint(0, 1 << 20, (N, 5), device="cuda", generator=g, dtype=torch.int32)]
    out = ops.compact_rows(ts, keep)
    for a, t in zip(out, ts):
        assert a.dtype == t.dtype and torch.equal(a, t[keep])
    many = [torch.randn(N, 2, device="cuda", generator=g) for _ in range(30)]   # more than one launch's worth
    for a, t in zip(ops.compact_rows(many, keep), many):
        assert torch.equal(a, t[keep])


def test_scene_prune_keeps_parameters_moments_and_trains_on():
    from fsgs import workloads as wl
    from fsgs.scene import DynamicScene, motion_at
    W, H, P = 160, 120, 6000
    surf = wl.surfels(P, seed=5, log_scale_mean=-2.5)
    sp = wl.superpoints(surf["means"], M=64, seed=1)
    cam = {k: v.cuda() for k, v in wl.camera(W, H).items()}
    motion = motion_at(sp, sp["centres"], "cuda")
    g = torch.Generator().manual_seed(9)
    g_img, g_op = torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()
    scene = DynamicScene(surf, sp["centres"], K=3, device="cuda")
    for _ in range(2):
        scene.train_step(cam, (W, H), motion, g_img, g_op)
    remove = (torch.rand(P, generator=g) < 0.4).cuda()
    before = [p.detach().clone() for p in scene.params]
    moments = [(scene.optimizer.state[p]["exp_avg"].clone(), scene.optimizer.state[p]["exp_avg_sq"].clone(),
                float(scene.optimizer.state[p]["step"])) for p in scene.params]
    idx_before, w_before = scene.knn_idx.clone(), scene.knn_w.clone()
    n = scene.prune(remove)
    keep = ~remove
    assert n == int(keep.sum()) == scene.num_points
    for p, b, (m, v, t) in zip(scene.params, before, moments):
        assert torch.equal(p.detach(), b[keep])
        st = scene.optimizer.state[p]
        assert torch.equal(st["exp_avg"], m[keep]) and torch.equal(st["exp_avg_sq"], v[keep]) and float(st["step"]) == t
    assert torch.equal(scene.knn_idx, idx_before[keep]) and torch.equal(scene.knn_w, w_before[keep])
    assert [g["params"][0] for g in scene.optimizer.param_groups] == scene.params or all(
        a is b for a, b in zip([g["params"][0] for g in scene.optimizer.param_groups], scene.params))
    out = scene.train_step(cam, (W, H), motion, g_img, g_op)     # the pruned scene renders and steps
    assert out["radii"].shape[0] == n and bool(torch.isfinite(out["images"]).all())
    assert float(scene.optimizer.state[scene.xyz]["step"]) == 3.0
