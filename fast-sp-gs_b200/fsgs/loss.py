"""Image loss of the training step, fused: ``lambda_l1 * mean|image - target| + lambda_ssim * (1 - mean SSIM)``
(the reference's rgb + ssim terms: exps/d_nerf.yaml:64-65, losses/image_loss.py, losses/ssim.py:69-99) in one forward
kernel (map, derivative maps, both sums) and one backward kernel that writes dL/dimage in the [3,H,W] layout the
compositing backward reads."""
import torch

from . import ops
from ._lib import lib, check

C1, C2 = 0.01 ** 2, 0.03 ** 2


class _L1SSIM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, image, target, lambda_l1, lambda_ssim):
        ops._need(image.is_cuda and image.dtype == torch.float32 and image.shape == target.shape and image.dim() == 3,
                  "l1_ssim_loss: image and target must be float32 CUDA tensors [C,H,W] of equal shape")
        image, target = image.contiguous(), target.contiguous()
        C, H, W = image.shape
        maps = torch.empty(4, C, H, W, device=image.device, dtype=torch.float32)
        sums = torch.zeros(2, device=image.device, dtype=torch.float32)
        p = ops._ptr
        check(lib().fsgs_ssim_forward(1, C, H, W, C1, C2, p(image), p(target), p(maps[0]), p(maps[1]), p(maps[2]),
                                      p(maps[3]), p(sums), ops._stream()), "fsgs_ssim_forward")
        n = float(C * H * W)
        ctx.save_for_backward(image, target, maps)
        ctx.weights = (lambda_l1 / n, lambda_ssim / n)
        return lambda_l1 * (sums[1] / n) + lambda_ssim * (1.0 - sums[0] / n)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g_loss):
        image, target, maps = ctx.saved_tensors
        C, H, W = image.shape
        w_l1, w_ssim = ctx.weights
        g = float(g_loss) if g_loss.device.type == "cpu" else None
        out = torch.empty_like(image)
        p = ops._ptr
        if g is None:
            # upstream scale lives on the device: keep it there (no synchronisation), scale afterwards
            check(lib().fsgs_ssim_backward(1, C, H, W, C1, C2, p(image), p(target), None, -w_ssim, w_l1, p(maps[1]),
                                           p(maps[2]), p(maps[3]), p(out), ops._stream()), "fsgs_ssim_backward")
            out = out * g_loss
        else:
            check(lib().fsgs_ssim_backward(1, C, H, W, C1, C2, p(image), p(target), None, -w_ssim * g, w_l1 * g,
                                           p(maps[1]), p(maps[2]), p(maps[3]), p(out), ops._stream()),
                  "fsgs_ssim_backward")
        return out, None, None, None


def l1_ssim_loss(image, target, lambda_l1=0.8, lambda_ssim=0.2):
    """Scalar loss (device tensor) of a rendered ``image`` [C,H,W] against ``target``; differentiable in ``image``."""
    return _L1SSIM.apply(image, target, float(lambda_l1), float(lambda_ssim))


def l1_ssim_value_and_grad(image, target, lambda_l1=0.8, lambda_ssim=0.2):
    """(loss, dL/dimage) without autograd: two kernel launches.  ``dL/dimage`` is ready to be handed to
    ``torch.autograd.backward(images, grad)`` or to the compositing backward directly."""
    image, target = image.detach().contiguous(), target.contiguous()
    C, H, W = image.shape
    maps = torch.empty(4, C, H, W, device=image.device, dtype=torch.float32)
    sums = torch.zeros(2, device=image.device, dtype=torch.float32)
    grad = torch.empty_like(image)
    n = float(C * H * W)
    p = ops._ptr
    check(lib().fsgs_ssim_forward(1, C, H, W, C1, C2, p(image), p(target), p(maps[0]), p(maps[1]), p(maps[2]),
                                  p(maps[3]), p(sums), ops._stream()), "fsgs_ssim_forward")
    check(lib().fsgs_ssim_backward(1, C, H, W, C1, C2, p(image), p(target), None, -lambda_ssim / n, lambda_l1 / n,
                                   p(maps[1]), p(maps[2]), p(maps[3]), p(grad), ops._stream()),
          "fsgs_ssim_backward")
    return lambda_l1 * (sums[1] / n) + lambda_ssim * (1.0 - sums[0] / n), grad
