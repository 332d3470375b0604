"""GPU tests of the image-loss epilogue: SSIM operators (reference names) and the fused L1 + SSIM loss."""
import pytest
import torch

import oracle as orc
from util import cpu, load_golden, reference_ext, rel_l2

pytestmark = pytest.mark.gpu

C1, C2 = 0.01 ** 2, 0.03 ** 2


@pytest.fixture(scope="module")
def ops():
    from fsgs import ops
    return ops


def _images(B, C, H, W, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.rand(B, C, H, W, generator=g)
    b = (a + 0.2 * torch.randn(B, C, H, W, generator=g)).clamp(0, 1)
    return a.cuda(), b.cuda()


def test_fusedssim_golden(ops):
    g = load_golden("ssim.npz", "cuda")
    m, d1, d2, d3 = ops.fusedssim(C1, C2, g["img1"], g["img2"], True)
    assert float((m - g["ssim_map"]).abs().max()) < 1e-5
    gx = ops.fusedssim_backward(C1, C2, g["img1"], g["img2"], g["up"], d1, d2, d3)
    assert rel_l2(gx, g["g_img1"]) < 1e-5
    m2, e1, e2, e3 = ops.fusedssim(C1, C2, g["img1"], g["img2"], False)
    assert torch.equal(m2, m) and e1.numel() == 0 and e3.numel() == 0


@pytest.mark.parametrize("B,C,H,W", [(1, 3, 800, 800), (2, 1, 33, 65), (1, 3, 5, 7), (1, 2, 64, 32), (1, 3, 1014, 1352)])
def test_fusedssim_vs_oracle_and_reference(ops, B, C, H, W):
    a, b = _images(B, C, H, W, seed=H)
    m, d1, d2, d3 = ops.fusedssim(C1, C2, a, b, True)
    up = torch.randn(B, C, H, W, generator=torch.Generator().manual_seed(1)).cuda()
    gx = ops.fusedssim_backward(C1, C2, a, b, up, d1, d2, d3)
    if H * W <= 800 * 800:
        o = orc.ssim_forward(cpu(a), cpu(b))
        assert float((cpu(m) - o[0]).abs().max()) < 1e-5
        for mine, theirs in zip((d1, d2, d3), o[1:]):
            assert rel_l2(mine, theirs) < 1e-5
        assert rel_l2(gx, orc.ssim_backward(cpu(a), cpu(b), cpu(up), *o[1:])) < 1e-5
    ref = reference_ext()
    if ref is not None and hasattr(ref, "fusedssim"):
        rm, r1, r2, r3 = ref.fusedssim(C1, C2, a, b, True)
        rg = ref.fusedssim_backward(C1, C2, a, b, up, r1, r2, r3)
        torch.cuda.synchronize()
        assert float((m - rm).abs().max()) < 1e-5
        assert rel_l2(d1, r1) < 1e-5 and rel_l2(d2, r2) < 1e-5 and rel_l2(d3, r3) < 1e-5
        assert rel_l2(gx, rg) < 1e-5
    # properties that hold at any size: identical images give a map of ones; the map is symmetric in its arguments
    ones = ops.fusedssim(C1, C2, a, a, False)[0]
    assert float((ones - 1).abs().max()) < 1e-5
    assert float((ops.fusedssim(C1, C2, b, a, False)[0] - m).abs().max()) < 1e-5


def test_l1_ssim_loss_and_gradient(ops):
    from fsgs.loss import l1_ssim_loss, l1_ssim_value_and_grad
    a, b = _images(1, 3, 120, 160, seed=9)
    img = a[0].clone().requires_grad_()
    loss = l1_ssim_loss(img, b[0])
    loss.backward()
    lo, go = orc.l1_ssim_loss(cpu(a[0]), cpu(b[0]))
    assert abs(float(loss) - float(lo)) < 1e-5
    assert rel_l2(img.grad, go) < 1e-4
    v, g = l1_ssim_value_and_grad(a[0], b[0])
    assert abs(float(v) - float(loss)) < 1e-6 and rel_l2(g, img.grad) < 1e-6
    # against torch autograd on the plain formula (five padded convolutions)
    win = torch.tensor([torch.exp(torch.tensor(-(i - 5) ** 2 / (2 * 1.5 ** 2))) for i in range(11)])
    win = (win / win.sum()).cuda()
    w2 = (win[:, None] * win[None, :]).expand(3, 1, 11, 11).contiguous()
    x = a.clone().requires_grad_()
    conv = lambda t: torch.nn.functional.conv2d(t, w2, padding=5, groups=3)
    mu1, mu2 = conv(x), conv(b)
    s11, s22, s12 = conv(x * x) - mu1 * mu1, conv(b * b) - mu2 * mu2, conv(x * b) - mu1 * mu2
    ssim = ((2 * mu1 * mu2 + C1) * (2 * s12 + C2)) / ((mu1 * mu1 + mu2 * mu2 + C1) * (s11 + s22 + C2))
    ref_loss = 0.8 * (x - b).abs().mean() + 0.2 * (1 - ssim.mean())
    ref_loss.backward()
    assert abs(float(ref_loss) - float(loss)) < 1e-5 and rel_l2(img.grad, x.grad[0]) < 1e-4


def test_train_step_with_loss_matches_autograd_route():
    """The fused step (loss kernels hand the image gradient to the compositing backward) equals rendering, calling
    the differentiable loss and letting autograd walk back."""
    from fsgs import workloads as wl
    from fsgs.loss import l1_ssim_loss
    from fsgs.scene import DynamicScene, motion_at
    W, H, P = 160, 120, 5000
    surf = wl.surfels(P, seed=5, log_scale_mean=-2.5)
    sp = wl.superpoints(surf["means"], M=64, seed=1)
    cam = {k: v.cuda() for k, v in wl.camera(W, H).items()}
    motion = motion_at(sp, sp["centres"], "cuda")
    target = torch.rand(3, H, W, generator=torch.Generator().manual_seed(2)).cuda()
    a, b = (DynamicScene(surf, sp["centres"], K=3, device="cuda") for _ in range(2))
    losses = []
    for _ in range(3):
        out, loss = a.train_step_with_loss(cam, (W, H), motion, target)
        losses.append(float(loss))
        out_b = b.render(cam, (W, H), motion)
        l1_ssim_loss(out_b["images"], target).backward()
        b.optimizer.set_before_step(out_b["visibility_filter"], P)
        b.optimizer.step()
        b.optimizer.zero_grad(set_to_none=True)
    assert all(l == l and l > 0 for l in losses) and losses[-1] < losses[0]
    # same kernels on both routes; float atomics in the compositing backward make the gradients differ in their last
    # bits, which Adam (steps of up to lr = 0.05 whatever the gradient's size) can amplify for a few elements
    for x, y in zip(a.params, b.params):
        d = (x - y).abs()
        assert float(d.mean()) < 1e-6 and float(d.max()) < 5e-4
