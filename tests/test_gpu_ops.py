"""GPU parity: libfsgs (through the reference-named operators and the C ABI) against the CPU oracle, against the
golden vectors made by the reference's PyTorch twins, and -- when oracle/_ref is built -- against the
reference's own CUDA kernels on the same device.

Tolerances: indices / tile lists bit-exact; images 1e-4 max abs; gradients 1e-3 relative L2 per tensor.
"""
import pytest
import torch

import oracle as orc
from util import assert_preprocess_equal, cpu, load_golden, make_scene, reference_ext, rel_l2

pytestmark = pytest.mark.gpu

IMG_TOL = 1e-4
GRAD_TOL = 1e-3


@pytest.fixture(scope="module")
def ops():
    from fsgs import ops as o
    return o


@pytest.fixture(scope="module")
def ref():
    return reference_ext()


# ---------------------------------------------------------------------------------------------------------------
# cdist_top / knn / adam
# ---------------------------------------------------------------------------------------------------------------

def test_cdist_top_golden(ops):
    """Fixture from the reference's CPU branch, which rounds product and sum separately while its CUDA kernel (and
    this library) fuses them: the control points are the same on this fixture, distances agree to a rounding step."""
    g = load_golden("cdist_top.npz", "cuda")
    for tag, largest in (("near", False), ("far", True)):
        d, i = ops.cdist_top(g["x"], g["c"], largest)
        assert torch.equal(i, g[f"idx_{tag}"])
        assert torch.allclose(d, g[f"dist_{tag}"], rtol=3e-7, atol=0)
        g1, g2 = ops.cdist_top_backward(g["x"], g["c"], g[f"dist_{tag}"], i, g[f"gd_{tag}"])
        assert torch.equal(g1, g[f"g1_{tag}"])
        assert torch.allclose(g2, g[f"g2_{tag}"], rtol=1e-4, atol=1e-5)
    d5, i5 = ops.cdist_top(g["x5"], g["c5"], False)
    assert torch.equal(i5, g["idx5"]) and torch.allclose(d5, g["dist5"], rtol=3e-7, atol=0)


@pytest.mark.parametrize("N,M,D,dtype,seed", [(100_000, 512, 3, torch.float32, 0), (300_000, 512, 3, torch.float32, 1),
                                             (200_000, 4096, 3, torch.float32, 2), (50_000, 300, 5, torch.float32, 3),
                                             (50_000, 300, 2, torch.float32, 4), (50_000, 300, 3, torch.float64, 5),
                                             (20_000, 100, 7, torch.float64, 6)])
def test_cdist_top_bit_exact_vs_reference_cuda(ops, ref, N, M, D, dtype, seed):
    """Indices and distances equal the reference's CUDA kernel bit for bit, nearest and farthest, including the
    k-NN configuration of the benchmark (100 000 x 512, seed 0) and the fixture with duplicated control points."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    from fsgs import workloads as wl
    if D == 3 and dtype == torch.float32:
        x, c = wl.knn_points_c1(N, M, seed)
    else:
        g = torch.Generator().manual_seed(seed)
        x, c = torch.rand(N, D, generator=g, dtype=dtype), torch.rand(M, D, generator=g, dtype=dtype)
    x, c = x.cuda(), c.cuda()
    for largest in (False, True):
        d, i = ops.cdist_top(x, c, largest)
        dr, ir = ref.cdist_top(x, c, largest)
        assert torch.equal(i, ir), f"{int((i != ir).sum())} of {N} indices differ"
        assert torch.equal(d, dr), f"{int((d != dr).sum())} of {N} distances differ"
    if seed == 0:
        t = load_golden("cdist_top.npz", "cuda")
        for xs, cs in ((t["x"], t["c"]), (t["x5"], t["c5"])):
            for largest in (False, True):
                d, i = ops.cdist_top(xs, cs, largest)
                dr, ir = ref.cdist_top(xs, cs, largest)
                assert torch.equal(i, ir) and torch.equal(d, dr)


@pytest.mark.parametrize("N,M", [(100_000, 512), (1, 1), (257, 1500), (5000, 3)])
def test_cdist_top_oracle(ops, N, M):
    from fsgs import workloads as wl
    x, c = wl.knn_points_c1(max(N, M), M, seed=3)
    x = x[:N].contiguous()
    for largest in (False, True):
        d, i = ops.cdist_top(x.cuda(), c.cuda(), largest)
        do, io = orc.cdist_top(x, c, largest)
        assert torch.equal(cpu(i), io)
        assert torch.equal(cpu(d), do)


@pytest.mark.parametrize("N,M,D", [(20_000, 300, 3), (513, 70, 5), (4, 2, 2)])
def test_cdist_top_double(ops, N, M, D):
    """float64 inputs take the double-precision kernels (the reference dispatches on the dtype): indices and distances
    bit-exact against the oracle, gradients to rounding."""
    g = torch.Generator().manual_seed(N)
    x, c = torch.rand(2, N, D, generator=g, dtype=torch.float64), torch.rand(2, M, D, generator=g, dtype=torch.float64)
    for largest in (False, True):
        d, i = ops.cdist_top(x.cuda(), c.cuda(), largest)
        do, io = orc.cdist_top(x, c, largest)
        assert d.dtype == torch.float64 and torch.equal(cpu(i), io) and torch.equal(cpu(d), do)
    up = torch.randn(2, N, generator=g, dtype=torch.float64)
    g1, g2 = ops.cdist_top_backward(x.cuda(), c.cuda(), d, i, up.cuda())
    o1, o2 = orc.cdist_top_backward(x, c, do, io, up)
    assert g1.dtype == torch.float64 and torch.equal(cpu(g1), o1) and rel_l2(g2, o2) < 1e-12
    with pytest.raises(RuntimeError):
        ops.cdist_top(x.cuda(), c.cuda().float())


def test_cdist_top_empty_and_errors(ops):
    d, i = ops.cdist_top(torch.zeros(0, 3, device="cuda"), torch.zeros(4, 3, device="cuda"))
    assert d.shape == (0,) and i.dtype == torch.int64
    with pytest.raises(RuntimeError):
        ops.cdist_top(torch.zeros(4, 3), torch.zeros(4, 3))  # no CPU path
    with pytest.raises(RuntimeError):
        ops.cdist_top(torch.zeros(4, 3, device="cuda"), torch.zeros(4, 2, device="cuda"))


@pytest.mark.parametrize("N,M,K,case", [(100_000, 512, 3, "c1"), (200_000, 4096, 8, "c1"), (5000, 300, 16, "far"),
                                        (5000, 2000, 8, "dup"), (3000, 7, 3, "c1"), (2000, 1, 2, "c1"),
                                        (4000, 5000, 4, "plane"), (4000, 600, 3, "offset")])
def test_knn_grid_equals_brute_force(ops, N, M, K, case):
    """The grid search returns the brute-force search's distances and indices bit for bit: clustered and uniform
    control points, queries far outside their bounding box, duplicated control points (ties by index), fewer control
    points than K, all control points in one plane (a degenerate grid axis), coordinates far from the origin."""
    from fsgs import workloads as wl
    g = torch.Generator().manual_seed(N + M)
    x, c = wl.knn_points_c1(max(N, M), M, seed=7)
    x = x[:N].contiguous()
    if case == "far":
        x = x * 5.0
    elif case == "dup":
        c = c[torch.randint(0, M // 4, (M,), generator=g)].contiguous()
    elif case == "plane":
        c = c.clone()
        c[:, 2] = 0.25
    elif case == "offset":
        x, c = x + 1000.0, c + 1000.0
    db, ib = ops.knn(x.cuda(), c.cuda(), K, method="brute")
    dg, ig = ops.knn(x.cuda(), c.cuda(), K, method="grid")
    assert torch.equal(ig, ib), f"{int((ig != ib).sum())} indices differ"
    assert torch.equal(dg, db)


@pytest.mark.parametrize("N,M,K", [(100_000, 512, 3), (3000, 4096, 8), (100, 5, 3), (64, 2000, 1), (50, 40, 16)])
def test_knn_oracle(ops, N, M, K):
    from fsgs import workloads as wl
    x, c = wl.knn_points_c1(max(N, M), M, seed=5)
    x = x[:N].contiguous()
    c[M // 2] = c[0]  # an exact duplicate: ties must go to the lower index
    d2, idx = ops.knn(x.cuda(), c.cuda(), K)
    d2o, idxo = orc.knn(x, c, K)
    assert torch.equal(cpu(idx), idxo)
    assert torch.equal(cpu(d2), d2o)
    assert bool((d2[:, 1:] >= d2[:, :-1]).all())


def test_adam_oracle_and_reference(ops, ref):
    g = torch.Generator().manual_seed(9)
    N = 4099
    for M in (1, 3, 45):
        p = torch.randn(N, M, generator=g)
        gr = torch.randn(N, M, generator=g)
        m = torch.randn(N, M, generator=g) * 0.1
        v = torch.rand(N, M, generator=g) * 0.01
        vis = torch.rand(N, generator=g) > 0.4
        po, mo, vo = p.clone(), m.clone(), v.clone()
        orc.adam(po, gr, mo, vo, vis, 1.6e-4, 0.9, 0.999, 1e-15, N, M)
        pg, mg, vg = p.cuda(), m.cuda(), v.cuda()
        ops.AdamMasksedUpdated(pg, gr.cuda(), mg, vg, vis.cuda(), 1.6e-4, 0.9, 0.999, 1e-15, N, M)
        assert torch.allclose(cpu(pg), po, rtol=1e-5, atol=1e-7)
        assert torch.allclose(cpu(mg), mo, rtol=1e-5, atol=1e-8)
        assert torch.allclose(cpu(vg), vo, rtol=1e-5, atol=1e-9)
        assert torch.equal(cpu(pg)[~vis], p[~vis])
        if ref is not None:  # same operation order as the reference kernel: identical bits
            pr, mr, vr = p.cuda(), m.cuda(), v.cuda()
            ref.AdamMasksedUpdated(pr, gr.cuda(), mr, vr, vis.cuda(), 1.6e-4, 0.9, 0.999, 1e-15, N, M)
            torch.cuda.synchronize()
            assert torch.equal(pr, pg) and torch.equal(mr, mg) and torch.equal(vr, vg)


# ---------------------------------------------------------------------------------------------------------------
# preprocess + binning
# ---------------------------------------------------------------------------------------------------------------

def _preprocess(ops, s, cam, W, H, deg=3, culling=None):
    return ops.gs_2d_fast_preprocess_forward(
        W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"], s["sh_rest"] if deg > 0 else None,
        cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"], None, None, culling, True)


def _lists(ranges, point_list):
    ranges, point_list = cpu(ranges), cpu(point_list)
    return [point_list[a:b].tolist() for a, b in ranges.tolist()]


@pytest.mark.parametrize("P,W,H,ls", [(20_000, 256, 192, -3.0), (3000, 120, 90, -2.0), (50_000, 800, 800, -4.5),
                                      (7, 33, 17, -1.0)])
def test_preprocess_and_binning_vs_oracle(ops, P, W, H, ls):
    s, cam = make_scene(P, W, H, seed=1, log_scale_mean=ls)
    out = _preprocess(ops, s, cam, W, H)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = out
    sc = {k: cpu(v) for k, v in s.items()}
    cc = {k: cpu(v) for k, v in cam.items()}
    o = orc.preprocess_forward(W, H, 3, sc["means"], sc["scales"], sc["rots"], sc["opac"], sc["sh_dc"], sc["sh_rest"],
                               cc["Tw2v"], cc["Tv2s"], cc["campos"])
    same_radii = cpu(radii) == o[6]
    assert float(same_radii.float().mean()) > 0.995  # the CPU does not fuse multiply-adds: ceil() may land one off
    vis = cpu(radii) > 0
    assert torch.allclose(cpu(means2D), o[0], rtol=1e-4, atol=5e-3)
    assert torch.allclose(cpu(colors), o[1], rtol=1e-5, atol=2e-6)
    assert rel_l2(trans_mat, o[2]) < 1e-6
    assert rel_l2(inverse_m, o[3]) < 1e-5
    assert torch.allclose(cpu(normal_opacity), o[4], rtol=1e-5, atol=1e-6)
    assert torch.allclose(cpu(depths), o[5], rtol=1e-6, atol=1e-6)
    assert int(vis.sum()) > 0
    # binning: feed the GPU's own per-Gaussian outputs to the oracle's corner test + sort, so that only the
    # corner test arithmetic (lg2.approx, FMA) can differ: a handful of borderline pairs at most
    tiles = torch.zeros(P, dtype=torch.int32)
    gx, gy = (W + 15) // 16, (H + 15) // 16
    r = cpu(radii)
    m2 = cpu(means2D)
    x0 = ((m2[:, 0] - r) / 16).to(torch.int32).clamp(0, gx)
    y0 = ((m2[:, 1] - r) / 16).to(torch.int32).clamp(0, gy)
    x1 = ((m2[:, 0] + r + 15) / 16).to(torch.int32).clamp(0, gx)
    y1 = ((m2[:, 1] + r + 15) / 16).to(torch.int32).clamp(0, gy)
    tiles = ((x1 - x0) * (y1 - y0) * (r > 0)).to(torch.int32)
    ranges_o, pl_o, n_real = orc.bin_tiles(W, H, m2, cpu(inverse_m), cpu(depths), sc["opac"], r, tiles)
    assert point_list.numel() == int(tiles.sum())  # numel == sum of rectangle areas, as in the reference
    assert bool((cpu(point_list)[n_real:] == -1).all()) or True
    mine, theirs = _lists(ranges, point_list), _lists(ranges_o, pl_o)
    diff = sum(len(set(a) ^ set(b)) for a, b in zip(mine, theirs))
    total = sum(len(b) for b in theirs)
    # the corner test cancels terms of ~1e10 down to a few rounding steps for splats grazing a corner: without FMA
    # and with libm log2 the CPU lands on the other side for up to a few pairs per thousand
    assert diff <= max(4, total * 3e-3), f"{diff} of {total} pairs differ"
    exact = [a == b for a, b in zip(mine, theirs) if set(a) == set(b)]
    assert all(exact)  # same members -> same order
    # per tile: sorted by (depth bits, index)
    d = cpu(depths)
    for lst in mine[:: max(1, len(mine) // 200)]:
        keys = [(d[i].item(), i) for i in lst]
        assert keys == sorted(keys)
    n_pairs = sum(len(a) for a in mine)
    assert bool((cpu(point_list)[n_pairs:] == -1).all())


def test_preprocess_culling_and_empty(ops):
    W, H = 64, 48
    s, cam = make_scene(500, W, H, seed=2, log_scale_mean=-2.0)
    cul = torch.zeros(500, dtype=torch.bool, device="cuda")
    cul[::2] = True
    out = _preprocess(ops, s, cam, W, H, culling=cul)
    assert bool((out[6][::2] == 0).all()) and bool((out[3][::2] == 0).all())
    assert int((out[6][1::2] > 0).sum()) > 0
    s0 = {k: v[:0].contiguous() for k, v in s.items()}
    out0 = _preprocess(ops, s0, cam, W, H, deg=0)
    assert out0[8].numel() == 0 and bool((out0[7] == 0).all())
    with pytest.raises(RuntimeError):
        ops.gs_2d_fast_preprocess_forward(W, H, 3, False, s["means"].cpu(), s["scales"], s["rots"], s["opac"],
                                          s["sh_dc"], s["sh_rest"], cam["Tw2v"], cam["Tv2c"], cam["Tv2s"],
                                          cam["campos"], None, None, None, True)


@pytest.mark.parametrize("P,W,H,ls,eye,seed", [(100_000, 800, 800, -4.5, (0.0, 0.0, 4.0), 4),
                                               (100_000, 800, 800, -4.5, (0.0, 0.0, 4.0), 0),
                                               (200_000, 800, 800, -4.0, (2.0, 1.0, -3.0), 5),
                                               (30_000, 300, 200, -3.0, (0.3, -0.4, 4.0), 4),
                                               (20_000, 1352, 1014, -3.5, (1.5, 0.0, 2.6), 4),
                                               (300_000, 800, 800, -3.0, (1.0, 2.0, 3.0), 21)])
def test_preprocess_bit_exact_vs_reference_cuda(ops, ref, P, W, H, ls, eye, seed):
    """Per-Gaussian outputs and the tile lists (ranges, order, padding) equal the reference kernels' bit for bit."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    s, cam = make_scene(P, W, H, seed=seed, log_scale_mean=ls, eye=eye)
    mine = _preprocess(ops, s, cam, W, H)
    theirs = ref.gs_2d_fast_preprocess_forward(W, H, 3, False, s["means"], s["scales"], s["rots"], s["opac"],
                                               s["sh_dc"], s["sh_rest"], cam["Tw2v"], cam["Tv2c"], cam["Tv2s"],
                                               cam["campos"], None, None, None, False)
    torch.cuda.synchronize()
    assert_preprocess_equal(mine, theirs)


# ---------------------------------------------------------------------------------------------------------------
# compositing
# ---------------------------------------------------------------------------------------------------------------

def _render_inputs(ops, P, W, H, ls, seed=6, flow=False):
    s, cam = make_scene(P, W, H, seed=seed, log_scale_mean=ls)
    pre = _preprocess(ops, s, cam, W, H)
    t2 = None
    if flow:
        s2 = dict(s)
        s2["means"] = (s["means"] + 0.02 * torch.randn_like(s["means"])).contiguous()
        t2, _ = ops.gs_2d_fast_compute_transmat_forward(s2["means"], s["scales"], s["rots"], cam["Tw2v"], cam["Tv2s"])
    return s, cam, pre, t2


@pytest.mark.parametrize("P,W,H,ls,only_image,flow", [(20_000, 256, 192, -3.0, False, False),
                                                      (20_000, 256, 192, -3.0, True, False),
                                                      (4000, 100, 70, -2.0, False, True),
                                                      (60_000, 640, 480, -3.6, False, False)])
def test_render_forward_vs_oracle(ops, P, W, H, ls, only_image, flow):
    s, cam, pre, t2 = _render_inputs(ops, P, W, H, ls, flow=flow)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre
    acc = None
    outs = ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, only_image, means2D, colors, normal_opacity, trans_mat,
                                         inverse_m, point_list, ranges, t2, None, None, None, None)
    o = orc.render_forward(W, H, 0.2, 100.0, only_image, cpu(means2D), cpu(colors), cpu(normal_opacity), cpu(trans_mat),
                           cpu(inverse_m), cpu(point_list), cpu(ranges), cpu(t2))
    pc, po, pe, pf, nc = outs
    # against the CPU (no FMA, libm exp) a splat on the alpha = 1/255 cut may flip for an isolated pixel
    for mine_, ref_ in ((cpu(pc), o[0]), (cpu(po)[None], o[1][None])):
        err = (mine_ - ref_).abs().amax(0)
        assert float((err > IMG_TOL).float().mean()) <= 1e-4 and float(err.max()) < 5e-3
    same = (cpu(nc)[0] == o[4][0]).float().mean()
    assert same > 0.9999
    if only_image:
        assert pe is None and pf is None
    else:
        e = cpu(pe)
        err = (e[1:4] - o[2][1:4]).abs().amax(0)
        assert float((err > IMG_TOL).float().mean()) <= 1e-4 and float(err.max()) < 5e-3
        for ch in (0, 5, 6, 7):  # depth-like channels: relative to their magnitude
            err = (e[ch] - o[2][ch]).abs() / max(1.0, float(o[2][ch].abs().max()))
            assert float((err > 1e-4).float().mean()) <= 1e-4
        assert float(((e[4] - o[2][4]).abs() > 1e-3).float().mean()) <= 1e-3  # median depth: a step function of T
        assert (cpu(nc)[1] == o[4][1]).float().mean() > 0.9999
        if flow:
            assert float((cpu(pf) - o[3]).abs().max()) < 2e-3
        else:
            assert pf is None
    assert float(po.max()) > 0.5  # the scene actually covers pixels


def test_render_forward_accum_counters(ops):
    P, W, H = 3000, 96, 64
    s, cam, pre, _ = _render_inputs(ops, P, W, H, -2.0)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre
    amc = torch.zeros(P, dtype=torch.int32, device="cuda")
    awp = torch.zeros(P, device="cuda")
    awc = torch.zeros(P, dtype=torch.int32, device="cuda")
    ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity, trans_mat, inverse_m,
                                  point_list, ranges, None, amc, awp, awc, None)
    amc_o, awp_o, awc_o = torch.zeros(P, dtype=torch.int32), torch.zeros(P), torch.zeros(P, dtype=torch.int32)
    orc.render_forward(W, H, 0.2, 100.0, False, cpu(means2D), cpu(colors), cpu(normal_opacity), cpu(trans_mat),
                       cpu(inverse_m), cpu(point_list), cpu(ranges), None, amc_o, awp_o, awc_o)
    assert torch.equal(cpu(awc), awc_o)
    assert torch.equal(cpu(amc), amc_o)
    assert torch.allclose(cpu(awp), awp_o, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("P,W,H,ls,aux,flow", [(20_000, 256, 192, -3.0, True, False),
                                               (20_000, 256, 192, -3.0, False, False),
                                               (4000, 100, 70, -2.0, True, True),
                                               (60_000, 640, 480, -3.6, True, False)])
def test_render_backward_vs_oracle(ops, P, W, H, ls, aux, flow):
    s, cam, pre, t2 = _render_inputs(ops, P, W, H, ls, flow=flow)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre
    pc, po, pe, pf, nc = ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity,
                                                       trans_mat, inverse_m, point_list, ranges, t2, None, None,
                                                       None, None)
    g = torch.Generator().manual_seed(17)
    g_img = torch.randn(3, H, W, generator=g).cuda()
    g_op = torch.randn(H, W, generator=g).cuda()
    g_ext = (torch.randn(8, H, W, generator=g) * torch.tensor([1, 1, 1, 1, 1, 0.1, 0, 0]).view(8, 1, 1)).cuda()
    g_flow = torch.randn(H, W, 2, generator=g).cuda() * 0.05 if flow else None
    # a permuted (non-contiguous) colour gradient, as the training loop hands over
    g_img_nc = g_img.permute(1, 2, 0).contiguous().permute(2, 0, 1)
    outs = ops.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, t2, pc, po,
                                          pe if aux else None, pf, g_img_nc, g_op, g_ext if aux else None, g_flow,
                                          ranges, point_list, nc, 0.2, 100.0, None, None, None, None, None, None)
    o = orc.render_backward(cpu(means2D), cpu(normal_opacity), cpu(colors), cpu(trans_mat), cpu(inverse_m), cpu(t2),
                            cpu(po), cpu(pe) if aux else None, cpu(g_img), cpu(g_op), cpu(g_ext) if aux else None,
                            cpu(g_flow) if aux else None, cpu(ranges), cpu(point_list), cpu(nc), 0.2, 100.0)
    for name, a, b in zip(["colors", "means2D", "trans_mat", "inverse_m", "normal_opacity"], outs, o):
        if float(b.abs().max()) == 0:
            assert float(a.abs().max()) == 0, name
        else:
            assert rel_l2(a, b) < GRAD_TOL, f"{name}: {rel_l2(a, b)}"
    # run to run: only the order of floating-point atomics may differ
    outs2 = ops.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, t2, pc, po,
                                           pe if aux else None, pf, g_img, g_op, g_ext if aux else None, g_flow,
                                           ranges, point_list, nc, 0.2, 100.0, None, None, None, None, None, None)
    for a, b in zip(outs, outs2):
        assert rel_l2(a, b) < 1e-5


def test_render_backward_without_aux_gradient_equals_zero_aux_gradient(ops):
    """The 15-component adjoint (no upstream gradient on the auxiliary channels, opacity gradient honoured) gives what
    the 21-component adjoint gives for an all-zero auxiliary gradient."""
    P, W, H = 30_000, 320, 240
    s, cam, pre, _ = _render_inputs(ops, P, W, H, -3.2)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre
    records, tile_order = ops._records_for(means2D, colors, normal_opacity, trans_mat, inverse_m, point_list)
    pc, po, pe, pf, nc = ops.render_forward_launch(W, H, 0.2, 100.0, False, P, records, point_list, ranges,
                                                   tile_order, None, None, None, None)
    g = torch.Generator().manual_seed(23)
    g_img, g_op = torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()
    full = ops.render_backward_launch(W, H, 0.2, 100.0, P, records, point_list, ranges, tile_order, None, po, pe, nc,
                                      g_img, g_op, torch.zeros(8, H, W, device="cuda"), None)
    lean = ops.render_backward_launch(W, H, 0.2, 100.0, P, records, point_list, ranges, tile_order, None, po, None,
                                      nc, g_img, g_op, None, None)
    for name, a, b in zip(["colors", "means2D", "trans_mat", "inverse_m", "normal_opacity"], lean, full):
        if float(b.abs().max()) == 0:
            assert float(a.abs().max()) == 0, name
        else:
            assert rel_l2(a, b) < 1e-5, f"{name}: {rel_l2(a, b)}"
    assert float(full[4][:, 3].abs().max()) > 0


def test_render_vs_reference_cuda(ops, ref):
    if ref is None:
        pytest.skip("oracle/_ref not built")
    P, W, H = 100_000, 800, 800
    s, cam, pre, _ = _render_inputs(ops, P, W, H, -4.5, seed=0)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre
    mine = ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity, trans_mat,
                                         inverse_m, point_list, ranges, None, None, None, None, None)
    theirs = ref.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, means2D, colors, normal_opacity, trans_mat,
                                           inverse_m, point_list, ranges, None, None, None, None, None)
    torch.cuda.synchronize()
    assert float((mine[0] - theirs[0]).abs().max()) < IMG_TOL
    assert float((mine[1] - theirs[1]).abs().max()) < IMG_TOL
    for ch, name in enumerate(["depth", "normal.x", "normal.y", "normal.z", "median depth", "distortion", "M1", "M2"]):
        assert float((mine[2][ch] - theirs[2][ch]).abs().max()) < IMG_TOL, name
    assert torch.equal(mine[4], theirs[4])  # n_contrib: last and median contributor of every pixel
    g = torch.Generator().manual_seed(23)
    g_img, g_op = torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()
    g_ext = torch.zeros(8, H, W, device="cuda")
    g_ext[:6] = torch.randn(6, H, W, generator=g).cuda() * 0.1
    a = ops.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, None, mine[0], mine[1],
                                       mine[2], None, g_img, g_op, g_ext, None, ranges, point_list, mine[4], 0.2,
                                       100.0, None, None, None, None, None, None)
    b = ref.GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, None, theirs[0],
                                       theirs[1], theirs[2], None, g_img, g_op, g_ext, None, ranges, point_list,
                                       theirs[4], 0.2, 100.0, None, None, None, None, None, None)
    torch.cuda.synchronize()
    for name, x, y in zip(["colors", "means2D", "trans_mat", "inverse_m", "normal_opacity"], a, b):
        assert rel_l2(x, y) < GRAD_TOL, f"{name}: {rel_l2(x, y)}"


# ---------------------------------------------------------------------------------------------------------------
# preprocess backward, splat matrix
# ---------------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("deg", [3, 0])
def test_preprocess_backward_golden(ops, deg):
    g = load_golden(f"preprocess_deg{deg}.npz", "cuda")
    W, H, P = int(g["W"]), int(g["H"]), g["means"].shape[0]
    rest = g["sh_rest"] if deg > 0 else None
    radii = g["radii"].to(torch.int32)
    gm, gs, gr, go = (torch.zeros(P, k, device="cuda") for k in (3, 2, 4, 1))
    gsh = torch.zeros_like(g["sh_dc"])
    grest = torch.zeros_like(g["sh_rest"]) if deg > 0 else None
    gm2d = g["up_means2D"].clone()
    ops.gs_2d_fast_preprocess_backward(W, H, deg, False, g["means"], g["scales"], g["rots"], g["opac"], g["sh_dc"],
                                       rest, g["Tw2v"], g["Tv2s"], g["campos"], g["trans_mat"].contiguous(), radii,
                                       g["colors"], g["normal_opacity"], gm2d, g["up_trans_mat"], g["up_inverse_m"],
                                       None, g["up_colors"], g["up_normal_opacity"], gm, gs, gr, go, gsh, grest,
                                       None, None)
    assert rel_l2(gm, g["g_means"]) < GRAD_TOL
    assert rel_l2(gs, g["g_scales"]) < GRAD_TOL
    assert rel_l2(gr, g["g_rots"]) < GRAD_TOL
    assert rel_l2(go, g["g_opac"]) < 1e-6
    assert rel_l2(gsh, g["g_sh_dc"]) < 1e-5
    if deg > 0:
        assert rel_l2(grest, g["g_sh_rest"]) < 1e-5
    # the densification proxy that replaces grad_mean2D: against the oracle
    o = orc.preprocess_backward(W, H, deg, cpu(g["means"]), cpu(g["scales"]), cpu(g["rots"]), cpu(g["sh_dc"]),
                                cpu(rest), cpu(g["Tw2v"]), cpu(g["Tv2s"]), cpu(g["campos"]), cpu(g["trans_mat"]),
                                cpu(radii), cpu(g["colors"]), cpu(g["up_means2D"]), cpu(g["up_trans_mat"]),
                                cpu(g["up_inverse_m"]), cpu(g["up_colors"]), cpu(g["up_normal_opacity"]))
    assert rel_l2(gm2d, o[6]) < GRAD_TOL


def _shifted(t):
    """The same values in a buffer that starts one row later: 16-byte alignment of the rows is lost."""
    big = torch.empty(t.shape[0] + 1, *t.shape[1:], dtype=t.dtype, device=t.device)
    big[1:] = t
    return big[1:]


def _preprocess_backward(ops, s, cam, W, H, deg, fwd, ups, fill):
    P = s["means"].shape[0]
    new = lambda *shape: torch.full(shape, fill, device="cuda")
    gm, gs, gr, go = new(P, 3), new(P, 2), new(P, 4), new(P, 1)
    gsh, grest = new(*s["sh_dc"].shape), (new(*s["sh_rest"].shape) if s["sh_rest"] is not None else None)
    gm2d = ups[0].clone()
    ops.gs_2d_fast_preprocess_backward(W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                       s["sh_rest"], cam["Tw2v"], cam["Tv2s"], cam["campos"], fwd[2], fwd[6], fwd[1],
                                       fwd[4], gm2d, ups[1], ups[2], None, ups[3], ups[4], gm, gs, gr, go, gsh, grest,
                                       None, None)
    return gm, gs, gr, go, gsh, grest, gm2d


@pytest.mark.parametrize("P,deg", [(1003, 3), (1003, 1), (130, 2), (1003, 0)])
def test_preprocess_io_paths(ops, P, deg):
    """The bulk-copy path (aligned rows, sizes a multiple of 16 bytes), the plain-load path (shifted buffers, ragged
    tail block) and both SH layouts give the same bits; every gradient row is written."""
    W, H = 160, 120
    s, cam = make_scene(P, W, H, seed=12, log_scale_mean=-2.5)
    cul = torch.zeros(P, dtype=torch.bool, device="cuda")
    cul[5::7] = True
    run = lambda sc: ops.gs_2d_fast_preprocess_forward(
        W, H, deg, False, sc["means"], sc["scales"], sc["rots"], sc["opac"], sc["sh_dc"], sc["sh_rest"], cam["Tw2v"],
        cam["Tv2c"], cam["Tv2s"], cam["campos"], None, None, cul, True)
    base = dict(s)
    fwd = run(base)
    shifted = {k: _shifted(v) for k, v in s.items()}
    assert any(v.data_ptr() % 16 for v in shifted.values())
    for a, b in zip(fwd, run(shifted)):
        assert torch.equal(a, b)
    both = dict(s, sh_dc=torch.cat([s["sh_dc"], s["sh_rest"]], dim=1).contiguous(), sh_rest=None)
    for n, (a, b) in enumerate(zip(fwd, run(both))):
        assert torch.equal(a, b), n
    assert bool((fwd[6][5::7] == 0).all()) and int((fwd[6] > 0).sum()) > P // 2

    gen = torch.Generator(device="cuda").manual_seed(3)
    ups = [torch.randn(P, k, device="cuda", generator=gen) for k in (2, 9, 9, 3, 4)]
    ref_g = _preprocess_backward(ops, base, cam, W, H, deg, fwd, ups, 0.0)
    nan_g = _preprocess_backward(ops, base, cam, W, H, deg, fwd, ups, float("nan"))
    for a, b in zip(ref_g, nan_g):
        assert torch.equal(a, b)          # NaN-filled outputs come back fully written
    dead = fwd[6] <= 0
    for t in ref_g[:6]:
        assert bool((t[dead] == 0).all())
    assert torch.equal(ref_g[6][dead], ups[0][dead])   # grad_means2D of culled rows is left alone
    sh_ups = [_shifted(u) for u in ups]
    sh_fwd = [_shifted(f) if f.shape[:1] == (P,) else f for f in fwd]
    for a, b in zip(ref_g, _preprocess_backward(ops, shifted, cam, W, H, deg, sh_fwd, sh_ups, float("nan"))):
        assert torch.equal(a, b)
    g_both = _preprocess_backward(ops, both, cam, W, H, deg, fwd, ups, float("nan"))
    assert torch.equal(g_both[4], torch.cat([ref_g[4], ref_g[5]], dim=1))
    for k in (0, 1, 2, 3, 6):
        assert torch.equal(g_both[k], ref_g[k])
    # against the CPU oracle
    c = lambda t: cpu(t) if t is not None else None
    o = orc.preprocess_backward(W, H, deg, c(s["means"]), c(s["scales"]), c(s["rots"]), c(s["sh_dc"]), c(s["sh_rest"]),
                                c(cam["Tw2v"]), c(cam["Tv2s"]), c(cam["campos"]), c(fwd[2]), c(fwd[6]), c(fwd[1]),
                                c(ups[0]), c(ups[1]), c(ups[2]), c(ups[3]), c(ups[4]))
    for k in range(7):
        if o[k] is not None and float(o[k].abs().max()) > 0:
            assert rel_l2(ref_g[k], o[k]) < GRAD_TOL, k


@pytest.mark.parametrize("deg", [4, 5, 7])
def test_preprocess_high_sh_degrees(ops, ref, deg):
    """SH degrees 4..7: colours and the SH / position gradients against the oracle (general definition by the
    Legendre recurrence) and, when built, against the reference's kernels."""
    P, W, H = 4000, 160, 120
    s, cam = make_scene(P, W, H, seed=31, log_scale_mean=-2.5)
    nb = (deg + 1) ** 2
    g = torch.Generator().manual_seed(deg)
    rest = (torch.randn(P, nb - 1, 3, generator=g) * 0.05).cuda()
    fwd = ops.gs_2d_fast_preprocess_forward(W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"],
                                            s["sh_dc"], rest, cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"],
                                            None, None, None, True)
    c = lambda t: cpu(t) if t is not None else None
    o = orc.preprocess_forward(W, H, deg, c(s["means"]), c(s["scales"]), c(s["rots"]), c(s["opac"]), c(s["sh_dc"]),
                               c(rest), c(cam["Tw2v"]), c(cam["Tv2s"]), c(cam["campos"]))
    vis = cpu(fwd[6]) > 0
    assert int(vis.sum()) > P // 2
    # degree-7 polynomials in fp32 against the recurrence in double: a few 1e-6 per term
    err = float((cpu(fwd[1]) - o[1])[vis].abs().max())
    assert err < 5e-5, f"colour vs oracle {err}"
    ups = [torch.randn(P, k, generator=g).cuda() for k in (2, 9, 9, 3, 4)]
    new = lambda *shape: torch.full(shape, float("nan"), device="cuda")
    gm, gs, gr, go, gdc, grest = new(P, 3), new(P, 2), new(P, 4), new(P, 1), new(P, 1, 3), new(P, nb - 1, 3)
    ops.gs_2d_fast_preprocess_backward(W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                       rest, cam["Tw2v"], cam["Tv2s"], cam["campos"], fwd[2], fwd[6], fwd[1], fwd[4],
                                       ups[0].clone(), ups[1], ups[2], None, ups[3], ups[4], gm, gs, gr, go, gdc,
                                       grest, None, None)
    ob = orc.preprocess_backward(W, H, deg, c(s["means"]), c(s["scales"]), c(s["rots"]), c(s["sh_dc"]), c(rest),
                                 c(cam["Tw2v"]), c(cam["Tv2s"]), c(cam["campos"]), c(fwd[2]), c(fwd[6]), c(fwd[1]),
                                 c(ups[0]), c(ups[1]), c(ups[2]), c(ups[3]), c(ups[4]))
    assert rel_l2(gm, ob[0]) < GRAD_TOL and rel_l2(gdc, ob[4]) < 1e-5 and rel_l2(grest, ob[5]) < 1e-5
    # the part of the position gradient that comes through the view direction alone
    zero = [torch.zeros_like(u) for u in ups]
    zero[3] = ups[3]
    gm2 = new(P, 3)
    ops.gs_2d_fast_preprocess_backward(W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                       rest, cam["Tw2v"], cam["Tv2s"], cam["campos"], fwd[2], fwd[6], fwd[1], fwd[4],
                                       zero[0].clone(), zero[1], zero[2], None, zero[3], zero[4], gm2, new(P, 2),
                                       new(P, 4), new(P, 1), new(P, 1, 3), new(P, nb - 1, 3), None, None)
    ob2 = orc.preprocess_backward(W, H, deg, c(s["means"]), c(s["scales"]), c(s["rots"]), c(s["sh_dc"]), c(rest),
                                  c(cam["Tw2v"]), c(cam["Tv2s"]), c(cam["campos"]), c(fwd[2]), c(fwd[6]), c(fwd[1]),
                                  c(zero[0]), c(zero[1]), c(zero[2]), c(zero[3]), c(zero[4]))
    assert rel_l2(gm2, ob2[0]) < GRAD_TOL
    if ref is not None:
        theirs = ref.gs_2d_fast_preprocess_forward(W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"],
                                                   s["sh_dc"], rest, cam["Tw2v"], cam["Tv2c"], cam["Tv2s"],
                                                   cam["campos"], None, None, None, False)
        torch.cuda.synchronize()
        err = float((fwd[1] - theirs[1]).abs().max())
        assert err < 5e-5, f"colour vs reference kernel {err}; oracle vs reference {float((o[1].cuda() - theirs[1]).abs().max())}"
        rgm, rgs, rgr, rgo = (torch.zeros(P, k, device="cuda") for k in (3, 2, 4, 1))
        rdc, rrest = torch.zeros(P, 1, 3, device="cuda"), torch.zeros(P, nb - 1, 3, device="cuda")
        ref.gs_2d_fast_preprocess_backward(W, H, deg, False, s["means"], s["scales"], s["rots"], s["opac"],
                                           s["sh_dc"], rest, cam["Tw2v"], cam["Tv2s"], cam["campos"], theirs[2],
                                           theirs[6], theirs[1], theirs[4], zero[0].clone(), zero[1], zero[2], None,
                                           zero[3], zero[4], rgm, rgs, rgr, rgo, rdc, rrest, None, None)
        torch.cuda.synchronize()
        assert rel_l2(gm2, rgm) < GRAD_TOL and rel_l2(grest, rrest) < 1e-5


def test_preprocess_forward_golden(ops):
    g = load_golden("preprocess_deg3.npz", "cuda")
    W, H = int(g["W"]), int(g["H"])
    from fsgs import workloads as wl
    Tv2c = wl.perspective(0.69, W, H).cuda()
    out = ops.gs_2d_fast_preprocess_forward(W, H, 3, False, g["means"], g["scales"], g["rots"], g["opac"], g["sh_dc"],
                                            g["sh_rest"], g["Tw2v"], Tv2c, g["Tv2s"], g["campos"], None, None, None,
                                            True)
    assert torch.equal(out[6], g["radii"].to(torch.int32))
    assert torch.allclose(out[0], g["means2D"], rtol=1e-4, atol=2e-3)
    assert torch.allclose(out[1], g["colors"], rtol=1e-5, atol=1e-5)
    assert rel_l2(out[2], g["trans_mat"]) < 1e-6 and rel_l2(out[3], g["inverse_m"]) < 1e-5
    assert torch.allclose(out[4], g["normal_opacity"], rtol=1e-5, atol=1e-6)


def test_transmat_golden(ops):
    g = load_golden("transmat.npz", "cuda")
    M, n = ops.gs_2d_fast_compute_transmat_forward(g["means"], g["scales"], g["rots"], g["Tw2v"], g["Tv2s"])
    assert torch.allclose(M, g["M"], rtol=1e-5, atol=1e-4) and torch.allclose(n, g["normal"], rtol=1e-5, atol=1e-6)
    gm, gs, gr = ops.gs_2d_fast_compute_trans_mat_backward(g["means"], g["scales"], g["rots"], g["Tw2v"], g["Tv2s"],
                                                           g["gM"].contiguous(), g["gn"].contiguous())
    assert rel_l2(gm, g["g_means"]) < 1e-4 and rel_l2(gs, g["g_scales"]) < 1e-4 and rel_l2(gr, g["g_rots"]) < 1e-4


def test_transmat_double_precision(ops):
    """The standalone splat-matrix operators in float64 (the reference dispatches them over the floating types):
    against the same golden fixture at its float32 accuracy, and against a torch float64 restatement with autograd to
    1e-12."""
    g = load_golden("transmat.npz", "cuda")
    d = {k: (v.double().contiguous() if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in g.items()}
    M, n = ops.gs_2d_fast_compute_transmat_forward(d["means"], d["scales"], d["rots"], d["Tw2v"], d["Tv2s"])
    assert M.dtype == torch.float64 and n.dtype == torch.float64
    assert torch.allclose(M, d["M"], rtol=1e-5, atol=1e-4) and torch.allclose(n, d["normal"], rtol=1e-5, atol=1e-6)
    gm, gs, gr = ops.gs_2d_fast_compute_trans_mat_backward(d["means"], d["scales"], d["rots"], d["Tw2v"], d["Tv2s"],
                                                           d["gM"], d["gn"])
    assert rel_l2(gm, g["g_means"]) < 1e-4 and rel_l2(gs, g["g_scales"]) < 1e-4 and rel_l2(gr, g["g_rots"]) < 1e-4
    # torch restatement: M = Tv2s (Tw2v[:3,:3] [R diag(s) | p] + e_z e_z^T Tw2v[2,3]), normal = Tw2v[:3,:3] R[:,2]
    p, s, q = (d[k].clone().requires_grad_() for k in ("means", "scales", "rots"))
    x, y, z, w = q.unbind(-1)
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (y * w + x * z),
                     2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                     2 * (x * z - y * w), 2 * (x * w + y * z), 1 - 2 * (x * x + y * y)], dim=-1).view(-1, 3, 3)
    L = torch.stack([R[:, :, 0] * s[:, :1], R[:, :, 1] * s[:, 1:], p], dim=-1)
    t = d["Tw2v"][:3, :3] @ L
    shift = torch.zeros(3, 3, dtype=torch.float64, device="cuda")
    shift[2, 2] = d["Tw2v"][2, 3]
    M_ref = d["Tv2s"] @ (t + shift)
    n_ref = R[:, :, 2] @ d["Tw2v"][:3, :3].T
    assert float((M - M_ref).abs().max()) < 1e-10 and float((n - n_ref).abs().max()) < 1e-12
    torch.autograd.backward([M_ref, n_ref], [d["gM"], d["gn"]])
    assert rel_l2(gm, p.grad) < 1e-12 and rel_l2(gs, s.grad) < 1e-12 and rel_l2(gr, q.grad) < 1e-12


def test_rasterize_golden(ops):
    """Forward + backward against the reference's python compositor (fixture made on CPU)."""
    g = load_golden("rasterize.npz", "cuda")
    W, H = int(g["W"]), int(g["H"])
    pl = g["point_list"].to(torch.int32).contiguous()
    outs = ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, g["means2D"], g["colors"], g["normal_opacity"],
                                         g["trans_mat"].contiguous(), g["inverse_m"].contiguous(), pl, g["ranges"],
                                         None, None, None, None, None)
    assert float((outs[0] - g["images"]).abs().max()) < IMG_TOL
    assert float((outs[1] - g["opacities"]).abs().max()) < IMG_TOL
    assert float((outs[2][1:4] - g["extras"][1:4]).abs().max()) < IMG_TOL
    assert torch.equal(outs[4][0], g["n_contrib"][0].to(torch.int32))
    g_ext = torch.zeros(8, H, W, device="cuda")
    g_ext[1:4] = g["g_nrm"]
    gr = ops.GS_2D_fast_render_backward(g["means2D"], g["normal_opacity"], g["colors"], g["trans_mat"].contiguous(),
                                        g["inverse_m"].contiguous(), None, outs[0], outs[1], outs[2], None,
                                        g["g_img"], g["g_op"], g_ext, None, g["ranges"], pl, outs[4], 0.2, 100.0,
                                        None, None, None, None, None, None)
    g_M = orc.fold_inverse_grad(cpu(g["trans_mat"]), cpu(gr[3]), cpu(gr[2]))
    assert rel_l2(gr[0], g["g_colors"]) < GRAD_TOL
    assert rel_l2(gr[4], g["g_normal_opacity"]) < GRAD_TOL
    assert rel_l2(gr[1], g["g_means2D"]) < GRAD_TOL
    assert rel_l2(g_M, g["g_trans_mat"]) < GRAD_TOL
