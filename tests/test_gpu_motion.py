"""The per-step superpoint motion operator (deformation network + warp head, kernel-weighted LBS weights) against
the fixture made by the reference's own module and against the CPU oracle (plain torch, fp32).

Tolerances: outputs 2e-5 max abs (the encodings reach sin(2^9 x): fp32 argument rounding dominates), parameter
gradients 1e-4 relative L2 per tensor.
"""
import pytest
import torch

import motion_oracle as mo
from util import load_golden, rel_l2

pytestmark = pytest.mark.gpu

OUT_TOL = 2e-5
GRAD_TOL = 1e-4
KEYS = ("sp_q", "sp_t", "sp_dr", "sp_ds")


def _reference_view(net, flat):
    """Named tensors in torch.nn.Linear orientation from a flat buffer laid out like ``net.params``."""
    v = net.views(flat)
    sd = {}
    for name, w in v.items():
        if name.startswith("heads"):
            continue
        sd[name] = w.t() if w.dim() == 2 else w
    hw, hb = v["heads.weight"], v["heads.bias"]
    for name, (lo, hi) in (("gaussian_warp", (0, 3)), ("gaussian_scaling", (3, 6)), ("gaussian_rotation", (6, 10)),
                           ("local_rotation", (10, 14))):
        if hi <= hw.shape[1]:
            sd[name + ".weight"], sd[name + ".bias"] = hw[:, lo:hi].t(), hb[lo:hi]
    return sd


def test_motion_matches_the_reference_network_fixture():
    from fsgs.motion import MotionNet
    g = load_golden("motion_w64.npz", "cuda")
    M = g["points"].shape[0]
    net = MotionNet(M, width=64, local_frame=True)
    net.load_reference_state_dict({k[len("param_"):]: v for k, v in g.items() if k.startswith("param_")})
    out = net.forward(g["points"].contiguous(), g["t"])
    for k in KEYS:
        assert float((out[k] - g["out_" + k]).abs().max()) < OUT_TOL, k
    g_params = torch.full_like(net.params.data, float("nan"))
    net.backward({k: g["up_" + k].contiguous() for k in KEYS}, g_params)
    got = _reference_view(net, g_params)                # NaN left anywhere in a section would show below
    for name, val in got.items():
        assert rel_l2(val, g["grad_" + name]) < GRAD_TOL, (name, rel_l2(val, g["grad_" + name]))


@pytest.mark.parametrize("M,width,local_frame,time_out", [(512, 256, True, 30), (512, 256, False, 30), (100, 128, True, 0),
                                                           (3, 32, True, 30)])
def test_motion_vs_oracle(M, width, local_frame, time_out):
    from fsgs.motion import MotionNet
    net = MotionNet(M, width=width, local_frame=local_frame, time_out=time_out, seed=3)
    gen = torch.Generator().manual_seed(M)
    with torch.no_grad():  # heads and biases that move something
        v = net.views()
        v["heads.weight"].copy_(torch.randn(v["heads.weight"].shape, generator=gen) * 0.05)
        v["heads.bias"].copy_(torch.randn(v["heads.bias"].shape, generator=gen) * 0.05)
        for i in range(net.cfg.depth):
            v[f"linear.{i}.bias"].copy_(torch.randn(width, generator=gen) * 0.1)
    pts = (torch.rand(M, 3, generator=gen) * 2 - 1).cuda()
    t = torch.tensor([0.61]).cuda()
    out = net.forward(pts, t)
    # The oracle runs in float64: with 2 million ReLUs per evaluation a pre-activation now and then lies within an
    # fp32 rounding of zero, and two fp32 summation orders then disagree on that unit's mask (seen: 4e-3 between the
    # oracle in fp32 and in fp64 on this very case).  Against fp64 the kernels measure 3e-7 to 5e-7.
    flat = net.params.detach().cpu().double().requires_grad_()
    ref = mo.motion(pts.cpu().double(), t.cpu().double(), _reference_view(net, flat), local_frame=local_frame)
    for k in KEYS:
        assert float((out[k].cpu() - ref[k].detach()).abs().max()) < OUT_TOL, k
    ups = {k: torch.randn(ref[k].shape, generator=gen) for k in KEYS}
    live = [k for k in KEYS if ref[k].requires_grad]    # without the fourth head sp_q is the constant (0, 0, 0, 1)
    torch.autograd.backward([ref[k] for k in live], [ups[k].double() for k in live])
    g_params = torch.full_like(net.params.data, float("nan"))
    net.backward({k: ups[k].cuda() for k in KEYS}, g_params)
    torch.cuda.synchronize()
    pad = torch.ones_like(g_params, dtype=torch.bool)   # the padding between sections is never written
    for name, off, n_in, n_out in net.sections():
        pad[off:off + max(n_in, 1) * n_out] = False
    assert bool(torch.isfinite(g_params[~pad]).all())
    mine, theirs = net.views(g_params), net.views(flat.grad.float().cuda())
    for name in mine:
        r = rel_l2(mine[name], theirs[name])
        assert r < GRAD_TOL or float(theirs[name].abs().max()) == 0, (name, r)
    # accumulate adds
    twice = g_params.clone()
    net.backward({k: ups[k].cuda() for k in KEYS}, twice, accumulate=True)
    assert rel_l2(twice[~pad], 2 * g_params[~pad]) < 1e-6


@pytest.mark.parametrize("P,M,K,with_weight", [(20_000, 512, 3, True), (5000, 64, 8, False)])
def test_kernel_weights_vs_oracle(P, M, K, with_weight):
    from fsgs import ops
    from fsgs.motion import kernel_weights, kernel_weights_backward
    from fsgs.renderer import group_pairs_by_superpoint
    gen = torch.Generator().manual_seed(P)
    x, c = torch.rand(P, 3, generator=gen), torch.rand(M, 3, generator=gen)
    d2, idx = ops.knn(x.cuda(), c.cuda(), K)
    raw_r = (torch.randn(M, generator=gen) * 0.3 - 2.0)
    raw_w = torch.randn(M, generator=gen) if with_weight else None
    w = kernel_weights(d2, idx, raw_r.cuda(), None if raw_w is None else raw_w.cuda())
    rr = raw_r.clone().requires_grad_()
    rw = None if raw_w is None else raw_w.clone().requires_grad_()
    ref = mo.kernel_weights(d2.cpu(), idx.cpu(), rr, rw)
    assert float((w.cpu() - ref).abs().max()) < 1e-6
    up = torch.randn(P, K, generator=gen)
    ref.backward(up)
    g_r = torch.full((M,), float("nan"), device="cuda")
    g_w = torch.full((M,), float("nan"), device="cuda") if with_weight else None
    kernel_weights_backward(d2, idx, raw_r.cuda(), None if raw_w is None else raw_w.cuda(), up.cuda(),
                            group_pairs_by_superpoint(idx, M), g_r, g_w)
    assert rel_l2(g_r, rr.grad) < GRAD_TOL
    if with_weight:
        assert rel_l2(g_w, rw.grad) < GRAD_TOL


def test_scene_trains_the_motion_network_and_kernel_weights():
    """``train_views`` with a time per view: the network's and the kernel weights' gradients (summed over two views,
    through LBS adjoint -> motion operator / weight kernel) and the dense Adam step against the same iteration built
    from the torch oracle of the motion, the autograd render operator and torch's Adam."""
    from fsgs import workloads as wl
    from fsgs.motion import MotionNet
    from fsgs.scene import DynamicScene
    W, H, P, M = 160, 120, 5000, 64
    surf = wl.surfels(P, seed=5, log_scale_mean=-3.2)
    centres = wl.superpoints(surf["means"], M=M, seed=1)["centres"]
    cams = [{k: v.cuda() for k, v in wl.camera(W, H, eye=e).items()} for e in ((0.0, 0.0, 4.0), (1.0, 0.5, 3.5))]
    gen = torch.Generator().manual_seed(9)
    ups = [(torch.randn(3, H, W, generator=gen).cuda(), torch.randn(H, W, generator=gen).cuda()) for _ in range(2)]
    ts = [torch.tensor([0.2]).cuda(), torch.tensor([0.7]).cuda()]
    raw_r, raw_w = torch.full((M,), -1.2), torch.randn(M, generator=gen) * 0.5

    def make():
        net = MotionNet(M, width=64, local_frame=True, seed=4)
        g2 = torch.Generator().manual_seed(5)
        with torch.no_grad():
            v = net.views()
            v["heads.weight"].copy_(torch.randn(v["heads.weight"].shape, generator=g2) * 0.02)
        return DynamicScene(surf, centres, K=3, device="cuda", motion_net=net, kernel_weights=(raw_r, raw_w),
                            lr_deform=1e-3), net

    a, net_a = make()
    b, net_b = make()
    torch_adam = torch.optim.Adam(b.dense_params, lr=1e-3, eps=1e-15)   # the autograd route steps with torch's own
    _, net_a_twin = make()   # same parameters as net_a before the step: supplies the native motion values to route b
    views = [dict(cam=cams[k], t=ts[k], g_images=ups[k][0], g_opacity=ups[k][1]) for k in (0, 1)]
    for _ in range(1):  # one iteration: the second already starts from parameters that differ by sign-like Adam steps
        a.train_views(views, (W, H))
        # the same iteration by autograd
        flat = net_b.params
        sd = _reference_view(net_b, flat)
        # values of the native kernels, derivatives of the oracle: the rendering is so sensitive to the motion (a shift
        # of 1e-7 moves splats across alpha and tile cuts) that the 1e-6 agreement of the two evaluations would
        # otherwise show up as per-mille noise in every gradient
        snap = lambda ref, native: ref + (native - ref).detach()
        b.knn_w = snap(mo.kernel_weights(b.knn_d2, b.knn_idx, b.sp_radius, b.sp_weight), a.knn_w)
        vis = None
        for k in (0, 1):
            native = net_a_twin.forward(b.centres, ts[k])
            motion = {n: snap(t, native[n]).contiguous()
                      for n, t in mo.motion(b.centres, ts[k], sd, local_frame=True).items()}
            out = b.render(cams[k], (W, H), motion)
            torch.autograd.backward([out["images"], out["opacity"]], list(ups[k]), retain_graph=(k == 0))
            vis = out["visibility_filter"] if vis is None else vis | out["visibility_filter"]
        b.optimizer.set_before_step(vis, P)
        b.optimizer.step()
        torch_adam.step()
        b.optimizer.zero_grad(set_to_none=True)
        torch_adam.zero_grad(set_to_none=True)
    a.check()
    from fsgs.scene import LRS
    lrs = [LRS[k] for k in ("xyz", "sh_dc", "sh_rest", "opacity", "scaling", "rotation")]
    for x, y, lr in zip(a.params, b.params, lrs):
        # the two routes evaluate the motion with different kernels (agreement 1e-5), and Adam turns a gradient that
        # is zero to rounding into a step of the full learning rate either way: a few elements may differ by up to
        # 2 lr, the mean by a small fraction of one step
        d = (x.detach() - y.detach()).abs()
        assert float(d.mean()) < 0.02 * lr + 1e-6 and float(d.max()) <= 2.1 * lr, (lr, float(d.mean()), float(d.max()))
    # dense parameters: they moved, and Adam's first moment -- linear in the gradient, unlike the parameters
    # themselves, whose first step is sign-like -- agrees to the noise of the float atomics in the compositing adjoint
    for x, y, x0 in ((net_a.params, net_b.params, MotionNet(M, width=64, local_frame=True, seed=4).params),
                     (a.sp_radius, b.sp_radius, raw_r.cuda()), (a.sp_weight, b.sp_weight, raw_w.cuda())):
        assert float((x.detach() - x0.detach().to(x.device)).abs().max()) > 1e-4
        ma, mb = a.dense_optimizer.state[x]["exp_avg"], torch_adam.state[y]["exp_avg"]
        assert rel_l2(ma, mb) < 1e-4, rel_l2(ma, mb)
        assert float((x.detach() - y.detach()).abs().mean()) < 0.1 * 1e-3
