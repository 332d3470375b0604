"""GPU tests of the host-side mirror: GS_2D_fast_render, the fused LBS warp, SparseGaussianAdam, install()."""
import sys

import pytest
import torch

import oracle as orc
from util import cpu, make_scene, rel_l2

pytestmark = pytest.mark.gpu


def _lbs_inputs(s, M=64, K=3, seed=0):
    from fsgs import ops, workloads as wl
    sp = wl.superpoints(s["means"].cpu(), M=M, seed=seed)
    c = sp["centres"].cuda()
    d2, idx = ops.knn(s["means"], c, K)
    w = torch.softmax(-d2, dim=-1).contiguous()
    q = sp["sp_q"].cuda()
    t = (sp["sp_t_raw"].cuda() + c - orc.quat_rotate(q, c)).contiguous()  # rotation about the superpoint's own centre
    return dict(xyz=s["means"], scaling_raw=s["log_scales"], rotation_raw=s["rots_raw"], knn_idx=idx, knn_w=w,
                sp_q=q, sp_t=t, sp_dr=sp["sp_dr"].cuda(), sp_ds=sp["sp_ds"].cuda())


@pytest.mark.parametrize("M", [64, 1024])   # 1024: the superpoint table no longer fits shared memory
def test_lbs_warp_forward_backward_vs_torch(M):
    from fsgs.renderer import lbs_warp
    s, cam = make_scene(5000, 64, 64, seed=3)
    L = _lbs_inputs(s, M=M)
    names = ["xyz", "scaling_raw", "rotation_raw", "knn_w", "sp_q", "sp_t", "sp_dr", "sp_ds"]
    a = {k: (v.clone().requires_grad_() if k in names else v) for k, v in L.items()}
    b = {k: (v.clone().requires_grad_() if k in names else v) for k, v in L.items()}
    order = ["xyz", "scaling_raw", "rotation_raw", "knn_idx", "knn_w", "sp_q", "sp_t", "sp_dr", "sp_ds"]
    out_a = lbs_warp(*[a[k] for k in order])
    out_b = orc.lbs_warp(*[b[k] for k in order])
    for x, y in zip(out_a, out_b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)
    g = torch.Generator().manual_seed(1)
    ups = [torch.randn(x.shape, generator=g).cuda() for x in out_a]
    torch.autograd.backward(out_a, ups)
    torch.autograd.backward(out_b, ups)
    for k in names:
        assert rel_l2(a[k].grad, b[k].grad) < 1e-4, k


def _render(s, cam, W, H, **kw):
    from fsgs.renderer import GS_2D_fast_render
    return GS_2D_fast_render(s.get("means"), s.get("scales"), s.get("rots"), s["opac"], (W, H), cam["Tw2v"],
                             cam["Tv2c"], cam["Tv2s"], cam["campos"], sh_degree=3, sh_features=s["sh_dc"],
                             sh_features_rest=s["sh_rest"], **kw)


def test_render_api_matches_operator_chain():
    from fsgs import ops
    P, W, H = 20_000, 256, 192
    s, cam = make_scene(P, W, H, seed=8)
    leaves = {k: s[k].clone().requires_grad_() for k in ("means", "scales", "rots", "opac", "sh_dc", "sh_rest")}
    out = _render(leaves, cam, W, H)
    assert set(out) >= {"images", "normals", "opacity", "distortion", "surf_depth", "surf_normal", "radii",
                        "viewspace_points", "visibility_filter", "flows"}
    assert out["images"].shape == (3, H, W) and out["surf_normal"].shape == (3, H, W) and out["flows"] is None
    pre = ops.gs_2d_fast_preprocess_forward(W, H, 3, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                            s["sh_rest"], cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"], None,
                                            None, None, True)
    fw = ops.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, pre[0], pre[1], pre[4], pre[2], pre[3], pre[8],
                                       pre[7], None, None, None, None, None)
    assert torch.equal(out["images"], fw[0]) and torch.equal(out["opacity"], fw[1])
    assert torch.equal(out["radii"], pre[6])
    g = torch.Generator().manual_seed(2)
    g_img, g_op = torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()
    (out["images"] * g_img).sum().backward(retain_graph=True)
    g1 = {k: v.grad.clone() for k, v in leaves.items()}
    gr = ops.GS_2D_fast_render_backward(pre[0], pre[4], pre[1], pre[2], pre[3], None, fw[0], fw[1], fw[2], None,
                                        g_img, torch.zeros_like(g_op), torch.zeros(8, H, W, device="cuda"), None,
                                        pre[7], pre[8], fw[4], 0.2, 100.0, None, None, None, None, None, None)
    gm, gs, gq, go = (torch.zeros(P, k, device="cuda") for k in (3, 2, 4, 1))
    gsh, grest = torch.zeros_like(s["sh_dc"]), torch.zeros_like(s["sh_rest"])
    ops.gs_2d_fast_preprocess_backward(W, H, 3, False, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"],
                                       s["sh_rest"], cam["Tw2v"], cam["Tv2s"], cam["campos"], pre[2], pre[6], pre[1],
                                       pre[4], gr[1], gr[2], gr[3], None, gr[0], gr[4], gm, gs, gq, go, gsh, grest,
                                       None, None)
    for k, ref in (("means", gm), ("scales", gs), ("rots", gq), ("opac", go), ("sh_dc", gsh), ("sh_rest", grest)):
        assert rel_l2(g1[k], ref) < 1e-4, k  # same kernels; only the order of float atomics differs
    assert rel_l2(out["viewspace_points"].grad, gr[1]) < 1e-4  # the densification proxy


def test_render_fused_lbs_equals_unfused():
    from fsgs.renderer import lbs_warp
    P, W, H = 20_000, 200, 160
    s, cam = make_scene(P, W, H, seed=9)
    L = _lbs_inputs(s, M=128)
    order = ["xyz", "scaling_raw", "rotation_raw", "knn_idx", "knn_w", "sp_q", "sp_t", "sp_dr", "sp_ds"]
    flt = [k for k in order if k != "knn_idx"]
    a = {k: (v.clone().requires_grad_() if k in flt else v) for k, v in L.items()}
    b = {k: (v.clone().requires_grad_() if k in flt else v) for k, v in L.items()}
    rest = {k: s[k] for k in ("opac", "sh_dc", "sh_rest")}
    out_a = _render(dict(rest), cam, W, H, lbs=[a[k] for k in order])
    m, sc, r = lbs_warp(*[b[k] for k in order])
    out_b = _render(dict(rest, means=m, scales=sc, rots=r), cam, W, H)
    assert torch.equal(out_a["images"], out_b["images"])
    g = torch.randn(3, H, W, generator=torch.Generator().manual_seed(4)).cuda()
    (out_a["images"] * g).sum().backward()
    (out_b["images"] * g).sum().backward()
    for k in flt:
        assert rel_l2(a[k].grad, b[k].grad) < 1e-4, k


def test_sparse_adam_fused_equals_per_tensor():
    from fsgs import ops
    from fsgs.optim import SparseGaussianAdam
    g = torch.Generator().manual_seed(5)
    N = 3001
    shapes = [(N, 3), (N, 1, 3), (N, 15, 3), (N, 1), (N, 2), (N, 4)]
    params = [torch.nn.Parameter(torch.randn(*sh, generator=g).cuda()) for sh in shapes]
    copies = [p.detach().clone() for p in params]
    lrs = [1.6e-4, 2.5e-3, 1.25e-4, 0.05, 5e-3, 1e-3]
    opt = SparseGaussianAdam([{"params": [p], "lr": lr} for p, lr in zip(params, lrs)], lr=0.0, eps=1e-15)
    ms = [torch.zeros_like(c) for c in copies]
    vs = [torch.zeros_like(c) for c in copies]
    for step in range(1, 4):
        vis = (torch.rand(N, generator=g) > 0.3).cuda()
        grads = [torch.randn(*sh, generator=g).cuda() for sh in shapes]
        for p, gr in zip(params, grads):
            p.grad = gr
        opt.set_before_step(vis, N)
        opt.step()
        for c, gr, m, v, lr in zip(copies, grads, ms, vs, lrs):
            t = torch.tensor(float(step), dtype=torch.float32)
            lr_eff = lr * (1 - 0.999 ** t) ** 0.5 / (1 - 0.9 ** t)
            ops.AdamMasksedUpdated(c, gr, m, v, vis, lr_eff, 0.9, 0.999, 1e-15, N, c.numel() // N)
        for p, c in zip(params, copies):
            assert torch.equal(p.detach(), c)
    assert opt.state[params[0]]["step"].item() == 3.0


def test_dense_adam_equals_torch_adam_and_obeys_its_gate():
    """``DenseAdam`` (dense tensors through the masked Adam kernel, one row each behind a one-element gate) against
    ``torch.optim.Adam`` over five steps; a gate <= 0 leaves parameters and moments alone."""
    from fsgs.optim import DenseAdam
    g = torch.Generator().manual_seed(2)
    shapes = [(523312,), (512,), (37, 5)]
    mine = [torch.nn.Parameter(torch.randn(s, generator=g).cuda()) for s in shapes]
    theirs = [torch.nn.Parameter(p.detach().clone()) for p in mine]
    a, b = DenseAdam(mine, lr=1e-3, eps=1e-15), torch.optim.Adam(theirs, lr=1e-3, eps=1e-15)
    for step in range(5):
        for p, q in zip(mine, theirs):
            grad = torch.randn(p.shape, generator=g).cuda() * (10.0 ** (step - 2))
            p.grad, q.grad = grad.clone(), grad.clone()
        a.step()
        b.step()
        for p, q in zip(mine, theirs):
            assert float((p.detach() - q.detach()).abs().max()) < 2e-6, step   # steps are ~1e-3: a few ulp of the update
            assert rel_l2(a.state[p]["exp_avg"], b.state[q]["exp_avg"]) < 1e-6
            # the kernel forms 1 - beta2 in float32 (as the reference's sparse Adam does), torch in double: 1.3e-5
            assert rel_l2(a.state[p]["exp_avg_sq"], b.state[q]["exp_avg_sq"]) < 3e-5
    before = [(p.detach().clone(), a.state[p]["exp_avg"].clone(), a.state[p]["exp_avg_sq"].clone()) for p in mine]
    for p in mine:
        p.grad = torch.ones_like(p)
    a.step(gate=torch.tensor([float("-inf")], device="cuda"))
    a.step(gate=torch.zeros(1, device="cuda"))
    for p, (p0, m0, v0) in zip(mine, before):
        assert torch.equal(p.detach(), p0) and torch.equal(a.state[p]["exp_avg"], m0)
        assert torch.equal(a.state[p]["exp_avg_sq"], v0)
    a.step(gate=torch.full((1,), 3.0, device="cuda"))
    assert not torch.equal(mine[0].detach(), before[0][0])


def test_install_exposes_the_reference_operator_names():
    import fsgs
    mod = fsgs.install("fast_2d_gs_test._C._C")
    names = ["gs_2d_fast_preprocess_forward", "gs_2d_fast_preprocess_backward", "GS_2D_fast_render_forward",
             "GS_2D_fast_render_backward", "gs_2d_fast_compute_transmat_forward",
             "gs_2d_fast_compute_trans_mat_backward", "cdist_top", "cdist_top_backward", "AdamMasksedUpdated",
             "fusedssim", "fusedssim_backward"]
    assert all(callable(getattr(mod, n)) for n in names)
    assert sys.modules["fast_2d_gs_test._C._C"] is mod

    class Holder:  # the reference stores operators as class attributes and calls them through self
        op = mod.cdist_top

    d, i = Holder().op(torch.rand(10, 3, device="cuda"), torch.rand(4, 3, device="cuda"))
    assert d.shape == (10,)


def test_list_overflow_is_reported():
    """A frame whose pairs do not fit the list buffer comes out as NaN (never as a plausible picture of truncated
    lists), the next render call of that size raises, and the capacity has grown by then."""
    from fsgs import renderer
    P, W, H = 20_000, 256, 192
    s, cam = make_scene(P, W, H, seed=8)
    key = (torch.cuda.current_device(), (P, W, H))
    saved = renderer._capacity.get(key)

    def starved():
        renderer._capacity[key] = renderer.ListCapacity(floor=16)
        renderer._capacity[key].high_water = 1  # pretend earlier frames of this size were almost empty
    try:
        starved()
        out = _render(s, cam, W, H, only_image=True)
        assert bool(torch.isnan(out["images"]).all()) and bool(torch.isnan(out["opacity"]).all())
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="overflowed"):
            renderer.check_overflow()
        out2 = _render(s, cam, W, H, only_image=True)  # capacity has grown: this frame is whole
        renderer.check_overflow()
        assert float(out2["opacity"].detach().max()) > 0.5
        # without an explicit check the NEXT render call of this size raises
        starved()
        _render(s, cam, W, H, only_image=True)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="overflowed"):
            _render(s, cam, W, H, only_image=True)
        # a frame size without history is sized exactly (one blocking read): no overflow, whole frame
        renderer._capacity[key] = renderer.ListCapacity(floor=16)
        out3 = _render(s, cam, W, H, only_image=True)
        renderer.check_overflow()
        assert torch.equal(out3["images"], out2["images"])
        # the training engine: same poison, same report
        from fsgs import workloads as wl
        from fsgs.scene import DynamicScene, motion_at
        surf = wl.surfels(P, seed=8, log_scale_mean=-3.0)
        sp = wl.superpoints(surf["means"], M=32, seed=1)
        scene = DynamicScene(surf, sp["centres"], K=3, device="cuda")
        eng = scene._engine((W, H))
        eng._reserve(16)
        eng.forward(scene, cam, motion_at(sp, sp["centres"], "cuda"))
        assert bool(torch.isnan(eng.images).all())
        with pytest.raises(RuntimeError, match="overflowed"):
            eng.check()
        eng.forward(scene, cam, motion_at(sp, sp["centres"], "cuda"))
        eng.check()
        assert bool(torch.isfinite(eng.images).all())
        # a training step on an overflowed view is dropped on the device: the view's backward writes -inf into the
        # mask, which no row of the masked Adam passes; the report comes with the next call
        before = {k: getattr(scene, k).detach().clone() for k in ("xyz", "opacity", "sh_dc", "scaling")}
        moments = scene.optimizer.state[scene.xyz]["exp_avg"].clone() if scene.xyz in scene.optimizer.state else None
        view = dict(cam=cam, motion=motion_at(sp, sp["centres"], "cuda"), g_images=torch.randn(3, H, W, device="cuda"),
                    g_opacity=torch.randn(H, W, device="cuda"))
        eng.high_water = 0
        eng._reserve(16)
        scene.train_views([view], (W, H))
        assert scene.last_step_dropped()
        for k, v in before.items():
            assert torch.equal(getattr(scene, k).detach(), v), k
        if moments is not None:
            assert torch.equal(scene.optimizer.state[scene.xyz]["exp_avg"], moments)
        with pytest.raises(RuntimeError, match="overflowed"):
            scene.check()
        scene.train_views([view], (W, H))   # capacity raised: this step counts
        scene.check()
        assert not scene.last_step_dropped()
        assert not torch.equal(scene.xyz.detach(), before["xyz"])
    finally:
        if saved is not None:
            renderer._capacity[key] = saved
        else:
            renderer._capacity.pop(key, None)


def test_epilogue_kernel_vs_torch_chain():
    """The fused epilogue against the reference's PyTorch operator chain (restated in fsgs.renderer), forward and
    backward."""
    from fsgs import renderer as R
    from fsgs import workloads as wl
    W, H = 200, 152
    cam = wl.camera(W, H, eye=(0.6, -0.5, 3.5), device="cuda")
    g = torch.Generator().manual_seed(3)
    extras = torch.rand(8, H, W, generator=g).cuda()
    extras[0] = extras[0] * 2 + 2
    extras[4] = extras[4] * 2 + 2
    extras[0, 5, 7] = float("nan")
    extras[4, 9, 3] = float("inf")
    opac = torch.rand(H, W, generator=g).cuda()
    ratio = 0.7
    a = extras.clone().requires_grad_()
    b = extras.clone().requires_grad_()
    n_a, sd_a, sn_a = R._SurfaceEpilogue.apply(a, opac, cam["Tw2v"], cam["Tv2c"], ratio)
    depths, normals, median, _d, _ = b.split([1, 3, 1, 1, 2], dim=0)
    n_b = (normals.permute(1, 2, 0) @ cam["Tw2v"][:3, :3]).permute(2, 0, 1)
    sd_b = torch.nan_to_num(depths, 0, 0) * (1 - ratio) + ratio * torch.nan_to_num(median, 0, 0)
    sn_b = R.depth_to_normal(cam["Tw2v"], cam["Tv2c"], (W, H), sd_b).permute(2, 0, 1) * opac
    assert torch.allclose(n_a, n_b, rtol=1e-5, atol=1e-6)
    assert torch.allclose(sd_a, sd_b, rtol=1e-6, atol=1e-6)
    assert float((sn_a - sn_b).abs().max()) < 2e-3 and rel_l2(sn_a, sn_b) < 1e-4
    ups = [torch.randn(t.shape, generator=g).cuda() for t in (n_a, sd_a, sn_a)]
    torch.autograd.backward([n_a, sd_a, sn_a], ups)
    torch.autograd.backward([n_b, sd_b, sn_b], ups)
    assert rel_l2(a.grad[1:4], b.grad[1:4]) < 1e-5
    assert rel_l2(a.grad[[0, 4]], b.grad[[0, 4]]) < 2e-3
    assert float(a.grad[5:].abs().max()) == 0


def test_host_feed_and_scalar_reader():
    """Buffered uploads arrive intact and in order; the scalar reader returns values one step late."""
    from fsgs.feed import HostFeed, ScalarReader
    feed, reader = HostFeed("cuda"), ScalarReader(lag=1)
    batches = [{"a": torch.full((1 << 20,), float(i)).pin_memory(),
                "n": {"b": torch.arange(8, dtype=torch.float32).add_(i).pin_memory()}} for i in range(6)]
    feed.stage(batches[0])
    got = []
    for i in range(6):
        if i + 1 < 6:
            feed.stage(batches[i + 1])
        x = feed.take()
        assert x["n"]["b"].data_ptr() % 256 == 0                # packed small tensors keep allocation alignment
        y = x["a"].sum() / x["a"].numel() + x["n"]["b"][0]      # consumes the buffers on the compute stream
        feed.release()
        reader.push(y)
        v = reader.pop()
        if v is not None:
            got.append(float(v))
    got += [float(v) for v in reader.drain()]
    assert got == [2.0 * i for i in range(6)]
    with pytest.raises(RuntimeError):
        feed.stage({"a": torch.zeros(1 << 20)})                 # large and not pinned
    feed2 = HostFeed("cuda", slots=2)
    feed2.stage(batches[0]); feed2.stage(batches[1])
    with pytest.raises(RuntimeError):
        feed2.stage(batches[2])                                 # both slots staged


def _autograd_step(scene, views, size):
    """The same iteration through the autograd operator: every view rendered and back-propagated (gradients add up in
    ``.grad``), visibility = union over the views, one optimiser step."""
    vis = None
    for v in views:
        out = scene.render(v["cam"], size, v["motion"])
        heads, grads = [out["images"]], [v["g_images"]]
        if v.get("g_opacity") is not None:
            heads.append(out["opacity"]), grads.append(v["g_opacity"])
        torch.autograd.backward(heads, grads)
        vis = out["visibility_filter"] if vis is None else vis | out["visibility_filter"]
    scene.optimizer.set_before_step(vis, scene.num_points)
    scene.optimizer.step()
    scene.optimizer.zero_grad(set_to_none=True)


def test_native_training_views_equal_the_autograd_route():
    """``train_views`` (two C calls per view, sigmoid and its adjoint inside the kernels, gradients of the views
    summed in place, float visibility mask) against rendering every view with the autograd operator: one view, two
    views, and the single-rank form of the multi-GPU step (split exchange)."""
    from fsgs import workloads as wl
    from fsgs.scene import DynamicScene, motion_at
    W, H, P = 160, 120, 5000
    surf = wl.surfels(P, seed=5, log_scale_mean=-2.5)
    sp = [wl.superpoints(surf["means"], M=64, seed=k) for k in (1, 2)]
    centres = sp[0]["centres"]
    cams = [{k: v.cuda() for k, v in wl.camera(W, H, eye=e).items()} for e in ((0.0, 0.0, 4.0), (1.0, 0.5, 3.5))]
    g = torch.Generator().manual_seed(9)
    views = [dict(cam=cams[k], motion=motion_at(sp[k], centres, "cuda"),
                  g_images=torch.randn(3, H, W, generator=g).cuda(), g_opacity=torch.randn(H, W, generator=g).cuda())
             for k in (0, 1)]
    for n_views, distributed in ((1, False), (2, False), (2, True)):
        a, b = (DynamicScene(surf, centres, K=3, device="cuda") for _ in range(2))
        for _ in range(2):
            a.train_views(views[:n_views], (W, H), distributed=distributed)
            _autograd_step(b, views[:n_views], (W, H))
        a.check()
        for x, y in zip(a.params, b.params):
            # not bit-equal: the compositing backward sums a Gaussian's tiles with float atomics in arrival order,
            # and Adam (steps of up to the learning rate whatever the gradient's size) amplifies that for a few elements
            d = (x - y).abs()
            assert float(d.mean()) < 1e-6 and float(d.max()) < 5e-4, (n_views, distributed)
    # a rank without a view this step (more ranks than views) steps with zero gradients and an empty mask: no change
    a = DynamicScene(surf, centres, K=3, device="cuda")
    a.train_views(views[:1], (W, H), distributed=True)
    before = [p.detach().clone() for p in a.params]
    a.train_views([], (W, H), distributed=True)
    assert all(torch.equal(p.detach(), q) for p, q in zip(a.params, before))
    # the sigmoid inside the preprocess kernel reproduces the framework's bits: identical radii and images
    a = DynamicScene(surf, centres, K=3, device="cuda")
    eng = a._engine((W, H))
    eng.forward(a, views[0]["cam"], views[0]["motion"])
    with torch.no_grad():
        out = a.render(views[0]["cam"], (W, H), views[0]["motion"])
    assert torch.equal(eng.radii, out["radii"]) and torch.equal(eng.images, out["images"])
    assert torch.equal(eng.opacity, out["opacity"])


def test_view_gradients_accumulate_in_call_order():
    """accumulate: the gradient buffers after views (v0, v1) hold g(v0) + g(v1) to rounding, the mask the union, and the
    superpoint-motion gradients those of the LAST view alone."""
    from fsgs import workloads as wl
    from fsgs.scene import DynamicScene, motion_at
    W, H, P = 160, 120, 4001
    surf = wl.surfels(P, seed=6, log_scale_mean=-2.5)
    sp = [wl.superpoints(surf["means"], M=64, seed=k) for k in (1, 2)]
    centres = sp[0]["centres"]
    cams = [{k: v.cuda() for k, v in wl.camera(W, H, eye=e).items()} for e in ((0.0, 0.0, 4.0), (2.5, 0.5, 2.0))]
    g = torch.Generator().manual_seed(1)
    ups = [(torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()) for _ in range(2)]
    s = DynamicScene(surf, centres, K=3, device="cuda")
    eng, b = s._engine((W, H)), s._grad_bucket()
    names = dict(xyz=s.xyz, scaling=s.scaling, rotation=s.rotation, opacity=s.opacity, sh_dc=s.sh_dc, sh_rest=s.sh_rest)

    def run(order, accumulate_from):
        dst = {k: torch.full_like(p, float("nan")) for k, p in names.items()}
        dst.update(visible=torch.full((P,), float("nan"), device="cuda"), knn_w=torch.full_like(s.knn_w, float("nan")),
                   **{k: torch.full_like(v, float("nan")) for k, v in s.motion_grads.items()})
        for j, k in enumerate(order):
            eng.forward(s, cams[k], motion_at(sp[k], centres, "cuda"))
            eng.backward(ups[k][0], ups[k][1], None, dst, accumulate=j >= accumulate_from)
        torch.cuda.synchronize()
        return dst

    g0, g1, both = run([0], 1), run([1], 1), run([0, 1], 1)
    for k in list(names) + ["knn_w"]:
        assert bool(torch.isfinite(both[k]).all()), k
        assert rel_l2(both[k], g0[k] + g1[k]) < 1e-5, k
    assert torch.equal(both["visible"], torch.maximum(g0["visible"], g1["visible"]))
    assert 0 < int(g0["visible"].sum()) < P or int(g0["visible"].sum()) == P
    for k in s.motion_grads:
        assert rel_l2(both[k], g1[k]) < 1e-5, k


def test_sh_gradient_rebuilt_from_its_factors():
    """The SH gradient of a view is (clamped colour gradient) x (SH basis of the view direction): the backward can hand
    out those six floats per Gaussian instead of the 48-float rows, and ``ops.sh_grad_from_views`` rebuilds the rows --
    bit-equal for one view, and for two views equal to the rows accumulated in the same order."""
    from fsgs import ops
    from fsgs import workloads as wl
    from fsgs.scene import DynamicScene, motion_at
    W, H, P = 160, 120, 4001
    surf = wl.surfels(P, seed=6, log_scale_mean=-2.5)
    sp = [wl.superpoints(surf["means"], M=64, seed=k) for k in (1, 2)]
    centres = sp[0]["centres"]
    cams = [{k: v.cuda() for k, v in wl.camera(W, H, eye=e).items()} for e in ((0.0, 0.0, 4.0), (2.5, 0.5, 2.0))]
    g = torch.Generator().manual_seed(1)
    ups = [(torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()) for _ in range(2)]
    s = DynamicScene(surf, centres, K=3, device="cuda")
    eng = s._engine((W, H))
    s._grad_bucket()  # creates the motion-gradient buffers
    names = dict(xyz=s.xyz, scaling=s.scaling, rotation=s.rotation, opacity=s.opacity, sh_dc=s.sh_dc, sh_rest=s.sh_rest)
    nan = lambda t: torch.full_like(t, float("nan"))
    rows = {k: nan(p) for k, p in names.items()}
    rows.update(visible=torch.zeros(P, device="cuda"), knn_w=nan(s.knn_w), **{k: nan(v) for k, v in s.motion_grads.items()})
    no_rows = dict(rows, sh_dc=None, sh_rest=None)
    no_rows.update({k: nan(names[k]) for k in ("xyz", "scaling", "rotation", "opacity")})
    factors = torch.full((3, P, 7), float("nan"), device="cuda")
    factors[2].zero_()  # an empty slot
    for j in (0, 1):
        eng.forward(s, cams[j], motion_at(sp[j], centres, "cuda"))
        eng.backward(ups[j][0], ups[j][1], None, rows, accumulate=j > 0, sh_source=factors[j])   # rows and factors
        if j == 0:
            first = {k: rows[k].clone() for k in ("sh_dc", "sh_rest")}
            alone = torch.full((P, 7), float("nan"), device="cuda")
            eng.backward(ups[j][0], ups[j][1], None, no_rows, sh_source=alone)                    # factors alone
            for k in ("xyz", "scaling", "rotation", "opacity"):  # equal up to the order of the compositing atomics
                assert rel_l2(no_rows[k], rows[k]) < 1e-6, k
            assert rel_l2(alone, factors[0]) < 1e-6
    # the same factors and mask from the early kernel (phase 3), the rest behind it (phase 4)
    early = torch.full((P, 7), float("nan"), device="cuda")
    split = dict(no_rows, visible=torch.full((P,), float("nan"), device="cuda"))
    split.update({k: nan(names[k]) for k in ("xyz", "scaling", "rotation", "opacity")})
    eng.backward(ups[1][0], ups[1][1], None, split, phase=3, sh_source=early)
    eng.backward(ups[1][0], ups[1][1], None, split, phase=4, sh_source=early)
    whole = dict(no_rows, visible=torch.full((P,), float("nan"), device="cuda"))
    whole.update({k: nan(names[k]) for k in ("xyz", "scaling", "rotation", "opacity")})
    late = torch.full((P, 7), float("nan"), device="cuda")
    eng.backward(ups[1][0], ups[1][1], None, whole, sh_source=late)
    assert rel_l2(early, late) < 1e-6 and torch.equal(split["visible"], whole["visible"])
    assert torch.equal(early[:, 6], whole["visible"]) and torch.equal(late[:, 6], whole["visible"])   # the seventh float
    for k in ("xyz", "scaling", "rotation", "opacity"):
        assert rel_l2(split[k], whole[k]) < 1e-4, k   # run-to-run order of the compositing atomics
    assert bool(torch.isfinite(factors).all())
    culled = eng.radii <= 0
    assert bool((factors[1][culled] == 0).all())
    dc, rest = nan(s.sh_dc), nan(s.sh_rest)
    ops.sh_grad_from_views(factors, [0], 3, dc, rest)
    assert torch.equal(dc, first["sh_dc"]) and torch.equal(rest, first["sh_rest"])
    seen = torch.full((P,), float("nan"), device="cuda")
    ops.sh_grad_from_views(factors, [0, 2, 1], 3, dc, rest, visible=seen)
    assert rel_l2(dc, rows["sh_dc"]) < 1e-6 and rel_l2(rest, rows["sh_rest"]) < 1e-6
    assert torch.equal(seen > 0, rows["visible"] > 0) and torch.equal(seen, factors[0][:, 6] + factors[1][:, 6])
    assert float(rest.abs().max()) > 0


@pytest.mark.parametrize("degree,n_rest,P", [(0, 15, 1000), (1, 15, 777), (2, 8, 130), (3, 15, 4097), (3, 0, 64)])
def test_sh_rows_from_factors_vs_the_oracle_basis(degree, n_rest, P):
    """``ops.sh_grad_from_views`` against sum_v basis(dir_v) x g_v formed with the oracle's SH basis, for every active
    degree, ragged sizes, slots in a given order and rows beyond the active degree left at zero."""
    from fsgs import ops
    g = torch.Generator().manual_seed(P)
    S = 3
    d = torch.nn.functional.normalize(torch.randn(S, P, 3, generator=g), dim=-1)
    c = torch.randn(S, P, 3, generator=g)
    c[1, ::3] = 0.0                                       # culled in that view: no contribution
    vis = (torch.rand(S, P, 1, generator=g) > 0.3).float()
    vis[2, 5] = float("-inf")                              # an overflowed view poisons the sum
    src = torch.cat([c, d, vis], dim=-1).contiguous().cuda()
    dc = torch.full((P, 1, 3), float("nan")).cuda()
    rest = torch.full((P, n_rest, 3), float("nan")).cuda() if n_rest else None
    seen = torch.full((P,), float("nan")).cuda()
    ops.sh_grad_from_views(src, [2, 0, 1], degree, dc, rest, visible=seen)
    assert torch.equal(seen.cpu(), vis[2, :, 0] + vis[0, :, 0] + vis[1, :, 0]) and float(seen[5]) == float("-inf")
    nb = (degree + 1) ** 2
    want = torch.zeros(P, 16, 3, dtype=torch.float64)
    for v in (2, 0, 1):
        b = orc.sh_basis(d[v], degree).double()           # [P, nb]
        want[:, :nb] += b[:, :, None] * c[v].double()[:, None, :]
    assert float((dc.cpu().double() - want[:, :1]).abs().max()) < 2e-6
    if n_rest:
        assert float((rest.cpu().double() - want[:, 1:1 + n_rest]).abs().max()) < 2e-6
        if nb - 1 < n_rest:
            assert bool((rest[:, nb - 1:] == 0).all())


@pytest.mark.parametrize("P", [3613, 4001, 130])
def test_training_step_with_odd_gaussian_counts(P):
    """Gaussian counts that are no multiple of 2 or 4: every per-Gaussian view of the flat gradient blocks (and of
    the communication bucket) must still start on an aligned address, since the kernels use float2 / float4 rows."""
    from fsgs import workloads as wl
    from fsgs.scene import DynamicScene, motion_at
    W, H = 160, 120
    surf = wl.surfels(P, seed=7, log_scale_mean=-2.5)
    sp = wl.superpoints(surf["means"], M=64, seed=1)
    cam = {k: v.cuda() for k, v in wl.camera(W, H).items()}
    motion = motion_at(sp, sp["centres"], "cuda")
    g = torch.Generator().manual_seed(3)
    g_img, g_op = torch.randn(3, H, W, generator=g).cuda(), torch.randn(H, W, generator=g).cuda()
    a, b = (DynamicScene(surf, sp["centres"], K=3, device="cuda") for _ in range(2))
    view = dict(cam=cam, motion=motion, g_images=g_img, g_opacity=g_op)
    for _ in range(2):
        out = a.train_step(cam, (W, H), motion, g_img, g_op, distributed=True)
        _autograd_step(b, [view], (W, H))
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out["images"]).all())
    for x, y in zip(a.params, b.params):
        d = (x - y).abs()
        assert float(d.mean()) < 1e-6 and float(d.max()) < 5e-4


@pytest.mark.parametrize("M,K", [(64, 3), (1024, 3), (4096, 8)])
def test_lbs_backward_grouped_pairs_equals_atomic_path_and_is_reproducible(M, K):
    """With the pairs grouped by superpoint the LBS adjoint sums each superpoint's row in one block: same values as the
    atomic path (to summation order), identical bits from run to run."""
    from fsgs.renderer import group_pairs_by_superpoint, lbs_backward
    s, cam = make_scene(20_000, 64, 64, seed=13)
    L = _lbs_inputs(s, M=M, K=K)
    order = ["xyz", "scaling_raw", "rotation_raw", "knn_idx", "knn_w", "sp_q", "sp_t", "sp_dr", "sp_ds"]
    ts = [L[k] for k in order]
    g = torch.Generator().manual_seed(5)
    ups = [torch.randn(20_000, n, generator=g).cuda() for n in (3, 2, 4)]
    pairs = group_pairs_by_superpoint(L["knn_idx"], M)
    flat = L["knn_idx"].reshape(-1)
    assert int(pairs[0][-1]) == flat.numel() and bool((flat[pairs[1].long()][1:] >= flat[pairs[1].long()][:-1]).all())
    plain = lbs_backward(ts, *ups)
    grouped = lbs_backward(ts, *ups, pairs=pairs)
    again = lbs_backward(ts, *ups, pairs=pairs)
    for a, b, c in zip(plain, grouped, again):
        assert rel_l2(a, b) < 1e-5
        assert torch.equal(b, c)
