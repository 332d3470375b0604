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
    flat = net.params.detach().cpu().clone().requires_grad_()
    ref = mo.motion(pts.cpu(), t.cpu(), _reference_view(net, flat), local_frame=local_frame)
    for k in KEYS:
        assert float((out[k].cpu() - ref[k].detach()).abs().max()) < OUT_TOL, k
    ups = {k: torch.randn(ref[k].shape, generator=gen) for k in KEYS}
    live = [k for k in KEYS if ref[k].requires_grad]    # without the fourth head sp_q is the constant (0, 0, 0, 1)
    torch.autograd.backward([ref[k] for k in live], [ups[k] for k in live])
    g_params = torch.full_like(net.params.data, float("nan"))
    net.backward({k: ups[k].cuda() for k in KEYS}, g_params)
    torch.cuda.synchronize()
    pad = torch.ones_like(g_params, dtype=torch.bool)   # the padding between sections is never written
    for name, off, n_in, n_out in net.sections():
        pad[off:off + max(n_in, 1) * n_out] = False
    assert bool(torch.isfinite(g_params[~pad]).all())
    mine, theirs = net.views(g_params), net.views(flat.grad)
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
