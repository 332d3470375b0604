"""Size-independent properties at the full sizes of the benchmark configurations (no CPU oracle runs at these
sizes): tile lists sorted and complete, forward deterministic, backward linear in the upstream gradient, optimiser
leaves invisible rows alone, k-NN exact."""
import pytest
import torch

from util import rel_l2

pytestmark = pytest.mark.gpu


def _scene(name, view=0):
    from fsgs import workloads as wl
    cfg = wl.CONFIGS[name]
    s = wl.surfels(cfg["P"], seed=0, log_scale_mean=cfg["log_scale_mean"], log_scale_std=cfg["log_scale_std"],
                   device="cuda")
    if "views" in cfg:
        eye = wl.arc_eye(cfg["radius"], view, cfg["views"])
    else:
        eye = (0.0, 0.0, 4.0)
    cam = {k: v.cuda() for k, v in wl.camera(cfg["W"], cfg["H"], eye=eye).items()}
    return cfg, s, cam


@pytest.mark.parametrize("name,view", [("train_300k_800", 0), ("multiview_500k_1352x1014", 5), ("stress_2m_1080p", 11)])
def test_lists_forward_backward_properties(name, view):
    from fsgs import ops
    cfg, s, cam = _scene(name, view)
    P, W, H = cfg["P"], cfg["W"], cfg["H"]
    pre = ops.gs_2d_fast_preprocess_forward(W, H, 3, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                            s["sh_rest"], cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"], None,
                                            None, None, True)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre
    T = ((W + 15) // 16) * ((H + 15) // 16)
    assert ranges.shape == (T, 2)
    # ranges tile the list front to back without gaps; the tail is padding
    lens = ranges[:, 1] - ranges[:, 0]
    assert bool((lens >= 0).all())
    nz = lens > 0
    starts = ranges[nz, 0]
    assert bool((starts[1:] == ranges[nz, 1][:-1]).all()) and int(starts[0]) == 0
    n_pairs = int(ranges[nz, 1][-1])
    assert n_pairs > P // 2 and bool((point_list[n_pairs:] == -1).all())
    body = point_list[:n_pairs].long()
    assert bool((body >= 0).all()) and bool((body < P).all()) and bool((radii[body] > 0).all())
    # inside every tile: ascending (depth bits, index), a Gaussian at most once
    tile_of = torch.repeat_interleave(torch.arange(T, device="cuda"), lens.clamp_min(0))
    key = (depths[body].view(torch.int32).long() << 32) | body
    same_tile = tile_of[1:] == tile_of[:-1]
    assert bool((key[1:][same_tile] > key[:-1][same_tile]).all())
    # number of pairs per Gaussian never exceeds its tile rectangle
    r = radii.float()
    gx, gy = (W + 15) // 16, (H + 15) // 16
    x0 = ((means2D[:, 0] - r) / 16).int().clamp(0, gx)
    x1 = ((means2D[:, 0] + r + 15) / 16).int().clamp(0, gx)
    y0 = ((means2D[:, 1] - r) / 16).int().clamp(0, gy)
    y1 = ((means2D[:, 1] + r + 15) / 16).int().clamp(0, gy)
    rect = ((x1 - x0) * (y1 - y0)).long() * (radii > 0)
    assert point_list.numel() == int(rect.sum())
    assert bool((torch.bincount(body, minlength=P) <= rect).all())

    # forward: deterministic, bounded
    fw = [ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity, trans_mat, inverse_m,
                                        point_list, ranges, None, None, None, None, None) for _ in range(2)]
    for a, b in zip(fw[0], fw[1]):
        if a is not None:
            assert torch.equal(a, b)
    img, op, ext, _, nc = fw[0]
    assert bool(torch.isfinite(img).all()) and bool(torch.isfinite(ext).all())
    assert float(op.min()) >= 0.0 and float(op.max()) <= 1.0
    tile_len = lens.view(gy, gx).repeat_interleave(16, 0).repeat_interleave(16, 1)[:H, :W]
    assert bool((nc[0] <= tile_len).all()) and bool((nc[1] <= nc[0]).all())
    assert bool(((nc[0] == 0) == (op == 0)).all())

    # backward: linear in the upstream gradient
    g = torch.Generator(device="cuda").manual_seed(5)
    ups = [(torch.randn(3, H, W, device="cuda", generator=g), torch.randn(H, W, device="cuda", generator=g),
            torch.randn(8, H, W, device="cuda", generator=g) * 0.1) for _ in range(2)]

    def bwd(u):
        return ops.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, None, img, op, ext,
                                              None, u[0], u[1], u[2], None, ranges, point_list, nc, 0.2, 100.0, None,
                                              None, None, None, None, None)

    ga, gb = bwd(ups[0]), bwd(ups[1])
    gab = bwd(tuple(2.0 * a - 0.5 * b for a, b in zip(ups[0], ups[1])))
    for x, y, z in zip(ga, gb, gab):
        assert bool(torch.isfinite(z).all())
        assert rel_l2(z, 2.0 * x - 0.5 * y) < 1e-3
    # no gradient for Gaussians that are in no list
    unused = torch.ones(P, dtype=torch.bool, device="cuda")
    unused[body] = False
    assert float(ga[0][unused].abs().max()) == 0 and float(ga[3][unused].abs().max()) == 0


def test_adam_touches_visible_rows_only_at_2m():
    from fsgs import ops
    N = 2_000_000
    g = torch.Generator(device="cuda").manual_seed(2)
    p = torch.randn(N, 15, 3, device="cuda", generator=g)
    grad, m, v = torch.randn_like(p), torch.zeros_like(p), torch.zeros_like(p)
    vis = torch.rand(N, device="cuda", generator=g) > 0.4
    p0 = p.clone()
    ops.AdamMasksedUpdated(p, grad, m, v, vis, 1e-3, 0.9, 0.999, 1e-15, N, 45)
    assert torch.equal(p[~vis], p0[~vis]) and float(m[~vis].abs().max()) == 0 and float(v[~vis].abs().max()) == 0
    # first step of Adam from zero moments: -lr * 0.1 g / (sqrt(0.001 g^2) + eps)
    step = (p - p0)[vis]
    want = -1e-3 * (0.1 * grad[vis]) / ((0.001 * grad[vis] ** 2).sqrt() + 1e-15)
    assert rel_l2(step, want) < 1e-4


def test_knn_exact_at_2m_points_4096_centres_k8():
    from fsgs import ops, workloads as wl
    x, c = wl.knn_points_c1(N=2_000_000, M=4096, seed=0)
    x, c = x.cuda(), c.cuda()
    d2, idx = ops.knn(x, c, 8)
    assert idx.dtype == torch.int64 and bool((idx >= 0).all()) and bool((idx < 4096).all())
    assert bool((d2[:, 1:] >= d2[:, :-1]).all())
    # the distances are those of the returned centres, by direct differences without fused multiply-adds
    diff = x[:, None, :] - c[idx]
    direct = (diff[..., 0] * diff[..., 0] + diff[..., 1] * diff[..., 1]) + diff[..., 2] * diff[..., 2]
    assert torch.equal(direct, d2)
    # exactness on a sample: nothing outside the returned set is closer than the 8th neighbour, ties broken by index
    sel = torch.randperm(x.shape[0], generator=torch.Generator().manual_seed(1))[:4000].cuda()
    dd = x[sel][:, None, :] - c[None]
    full = (dd[..., 0] * dd[..., 0] + dd[..., 1] * dd[..., 1]) + dd[..., 2] * dd[..., 2]
    order = torch.sort(full * 1.0, dim=1, stable=True)
    assert torch.equal(order.values[:, :8], d2[sel])
    assert torch.equal(order.indices[:, :8], idx[sel])
