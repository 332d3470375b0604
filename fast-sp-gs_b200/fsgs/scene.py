"""A minimal dynamic surfel scene: the parameters the reference model owns (``fast_2d_gs/network.py:357``:
positions, 2 log-scales, rotation, opacity logit, SH DC + 15 rest coefficients = 58 floats per Gaussian), the
superpoint k-NN / LBS weights (``network.py:498-521``, 'dist' weighting) and one training step
(warp -> render -> backward -> visibility-masked Adam) as ``train.py:343-412`` runs it, minus losses: the
upstream image gradient is an input.
"""
import torch

from . import ops
from .dist import GradBucket, reduce_visibility
from .optim import SparseGaussianAdam
from .renderer import GS_2D_fast_render, group_pairs_by_superpoint, list_capacity

# learning rates of exps/d_nerf.yaml (position lr at its initial value)
LRS = dict(xyz=1.6e-4, sh_dc=2.5e-3, sh_rest=1.25e-4, opacity=0.05, scaling=5e-3, rotation=1e-3)


def lbs_weights(d2, idx, mode="dist", temperature=1.0, radius=None, weight=None, table=None):
    """Blend weights [N,K] of each Gaussian's K nearest superpoints from the squared distances ``d2`` [N,K] and
    indices ``idx`` [N,K] of the k-NN search; the three forms of the reference's ``calc_LBS_weight``
    (fast_2d_gs/network.py:506-518):

    * ``"dist"``: softmax(-d2 / temperature);
    * ``"kernel"``: exp(-d2 / (2 r^2)) with the per-superpoint ``radius`` [M], times the per-superpoint ``weight`` [M]
      when given, plus 1e-7, normalised to sum 1 (the shipped configuration's 'weighted_kernel');
    * ``"table"``: softmax over the K gathered entries of a learned ``table`` [N,M].

    Plain torch operations on [N,K] tensors, differentiable in ``radius``, ``weight`` and ``table``."""
    if mode == "dist":
        return torch.softmax(-d2 / temperature, dim=-1)
    if mode == "kernel":
        r = radius[idx]
        w = torch.exp(-d2 / (2 * r ** 2))
        if weight is not None:
            w = w * weight[idx]
        w = w + 1e-7
        return w / w.sum(dim=-1, keepdim=True)
    if mode == "table":
        return torch.gather(table, dim=1, index=idx).softmax(dim=-1)
    raise ValueError(f"unknown LBS weighting {mode!r}")


class DynamicScene:
    def __init__(self, surfels, centres, K=3, eps=1e-15, device="cuda", lrs=None):
        P = lambda t: torch.nn.Parameter(t.to(device).contiguous())
        self.xyz = P(surfels["means"])
        self.scaling = P(surfels["log_scales"])
        self.rotation = P(surfels["rots_raw"])
        self.opacity = P(surfels["opac_raw"])
        self.sh_dc = P(surfels["sh_dc"])
        self.sh_rest = P(surfels["sh_rest"])
        self.centres = centres.to(device).contiguous()
        self.K = K
        self.refresh_knn()
        LRS = dict(globals()["LRS"], **(lrs or {}))
        groups = [dict(params=[self.xyz], lr=LRS["xyz"]), dict(params=[self.sh_dc], lr=LRS["sh_dc"]),
                  dict(params=[self.sh_rest], lr=LRS["sh_rest"]), dict(params=[self.opacity], lr=LRS["opacity"]),
                  dict(params=[self.scaling], lr=LRS["scaling"]), dict(params=[self.rotation], lr=LRS["rotation"])]
        self.optimizer = SparseGaussianAdam(groups, lr=0.0, eps=eps)
        self.bucket = None

    @property
    def params(self):
        return [self.xyz, self.sh_dc, self.sh_rest, self.opacity, self.scaling, self.rotation]

    @property
    def num_points(self):
        return self.xyz.shape[0]

    @torch.no_grad()
    def refresh_knn(self, mode="dist", **weighting):
        """K nearest superpoints of every Gaussian and their blend weights (``lbs_weights``; default softmax(-d^2))."""
        d2, idx = ops.knn(self.xyz.detach(), self.centres, self.K)
        self.knn_idx = idx
        self.knn_w = lbs_weights(d2, idx, mode, **weighting).contiguous()
        # pairs grouped by superpoint: the LBS adjoint then needs no atomics
        self.knn_idx.superpoint_pairs = group_pairs_by_superpoint(idx, self.centres.shape[0])

    def render(self, cam, size, motion, only_image=False, grad_out=None):
        """``motion``: dict sp_q [M,4] unit quaternions, sp_t [M,3], sp_dr [M,4], sp_ds [M,2] for this time step."""
        lbs = (self.xyz, self.scaling, self.rotation, self.knn_idx, self.knn_w, motion["sp_q"], motion["sp_t"],
               motion["sp_dr"], motion["sp_ds"])
        return GS_2D_fast_render(None, None, None, torch.sigmoid(self.opacity), size, cam["Tw2v"], cam["Tv2c"],
                                 cam["Tv2s"], cam["campos"], sh_degree=3, sh_features=self.sh_dc,
                                 sh_features_rest=self.sh_rest, lbs=lbs, only_image=only_image, grad_out=grad_out)

    def train_step(self, cam, size, motion, g_images, g_opacity, group=None, distributed=False, g_aux=None):
        """One iteration: forward, backward with the given upstream gradients on images [3,H,W] and opacity [H,W]
        (and, with ``g_aux = {"normals": [3,H,W], "distortion": [1,H,W], ...}``, on those entries of the render
        dictionary), (all-reduce of the gradients and of the visibility mask when ``distributed``), fused masked
        Adam.  Returns the render dictionary."""
        if not distributed:
            out = self.render(cam, size, motion)
            self._backward(out, g_images, g_opacity, g_aux)
            self.optimizer.set_before_step(out["visibility_filter"], self.num_points)
            self.optimizer.step_visible()
            self._drop_grads()
            return out
        # Multi-GPU.  Bucket segments: SH DC, SH rest, visibility mask | position, opacity, scale, rotation.
        # The backward kernels write into the bucket.  The first three segments (49 of the 59 floats per Gaussian)
        # are all-reduced as soon as the preprocess adjoint has been queued, beside the LBS adjoint; the rest follows;
        # Adam runs on the SH tensors while the second exchange is in flight.
        if self.bucket is None:
            self.bucket = GradBucket([self.sh_dc, self.sh_rest, self.xyz, self.opacity, self.scaling, self.rotation],
                                     extra=self.num_points, extra_after=1)
        b = self.bucket
        early = []
        grad_out = None
        if all(p.grad is None for p in self.params):
            grad_out = dict(sh_features=b.view_of(self.sh_dc), sh_features_rest=b.view_of(self.sh_rest),
                            xyz=b.view_of(self.xyz), scaling_raw=b.view_of(self.scaling),
                            rotation_raw=b.view_of(self.rotation),
                            on_sh_ready=lambda: early.append(b.reduce_span(0, 2, group)))
        out = self.render(cam, size, motion, grad_out=grad_out)
        b.extra.copy_(out["visibility_filter"])  # known after the forward: travels with the first exchange
        self._backward(out, g_images, g_opacity, g_aux)
        sh_in_place = all(p.grad is not None and p.grad.data_ptr() == b.view_of(p).data_ptr()
                          for p in (self.sh_dc, self.sh_rest))
        b.pack()  # copies in what the kernels did not write in place (the opacity gradient)
        if early and not sh_in_place:
            # autograd did not adopt the in-place SH gradients (it made copies, which pack() has just moved in): the
            # early exchange summed stale data; let it finish, then exchange those segments again from fresh contents
            if early[0] is not None:
                early[0].wait()
            b.extra.copy_(out["visibility_filter"])
            early = [b.reduce_span(0, 2, group)]
        if early:
            late = b.reduce_span(3, 6, group)
        else:  # gradients were not produced in place: one exchange for everything
            early.append(b.reduce_span(0, 6, group))
            late = None
        b.adopt()
        if early[0] is not None:
            early[0].wait()
        visible = b.extra > 0
        self.optimizer.set_before_step(visible, self.num_points)
        self.optimizer.step_visible(only=[self.sh_dc, self.sh_rest])
        if late is not None:
            late.wait()
        self.optimizer.step_visible(only=[self.xyz, self.opacity, self.scaling, self.rotation])
        self._drop_grads()
        return out

    def train_step_with_loss(self, cam, size, motion, target, lambda_l1=0.8, lambda_ssim=0.2, group=None,
                             distributed=False):
        """One iteration against a target image [3,H,W]: forward, fused L1 + SSIM loss and its image gradient
        (``fsgs.loss``), backward, optimiser.  Returns (render dictionary, loss as a device scalar)."""
        from .loss import l1_ssim_value_and_grad
        holder = {}

        def upstream(out):
            holder["loss"], g = l1_ssim_value_and_grad(out["images"], target, lambda_l1, lambda_ssim)
            return g

        out = self.train_step(cam, size, motion, upstream, None, group=group, distributed=distributed)
        return out, holder["loss"]

    @torch.no_grad()
    def prune(self, remove):
        """Drop the Gaussians whose entry in ``remove`` (bool [P]) is set: all six parameter tensors, both Adam moments
        of each and the superpoint neighbours are compacted together (``ops.compact_rows``); what the reference's
        ``prune_points`` does tensor by tensor (fast_2d_gs/gaussian_splatting.py:557-568).  Returns the new count."""
        keep = ~remove
        params = self.params
        moments = []
        for p in params:
            st = self.optimizer.state.get(p, {})
            moments += [st.get("exp_avg"), st.get("exp_avg_sq")]
        extra = [self.knn_idx, self.knn_w]
        rows = [p.data for p in params] + [m for m in moments if m is not None] + extra
        out = ops.compact_rows(rows, keep)
        new_params = [torch.nn.Parameter(t) for t in out[:len(params)]]
        rest = out[len(params):]
        for group, old, new in zip(self.optimizer.param_groups, params, new_params):
            st = self.optimizer.state.pop(old, None)
            group["params"][0] = new
            if st:
                st["exp_avg"], st["exp_avg_sq"] = rest.pop(0), rest.pop(0)
                self.optimizer.state[new] = st
        self.xyz, self.sh_dc, self.sh_rest, self.opacity, self.scaling, self.rotation = new_params
        self.knn_idx, self.knn_w = rest
        self.knn_idx.superpoint_pairs = group_pairs_by_superpoint(self.knn_idx, self.centres.shape[0])
        self.bucket = None
        return self.num_points

    def _drop_grads(self):
        for p in self.params:  # zero_grad(set_to_none=True) without the optimizer's hook and profiling layers
            p.grad = None

    def _backward(self, out, g_images, g_opacity, g_aux):
        if callable(g_images):  # the upstream image gradient is a function of the rendered result (a loss)
            g_images = g_images(out)
        if g_opacity is None:
            torch.autograd.backward([out["images"]], [g_images])
            return
        heads, grads = [out["images"], out["opacity"]], [g_images, g_opacity]
        for name, g in (g_aux or {}).items():
            heads.append(out[name])
            grads.append(g)
        torch.autograd.backward(heads, grads)

    def check(self):
        list_capacity(self.xyz.device).check_overflow()


def motion_at(sp, centres, device="cuda"):
    """Superpoint motion of ``workloads.superpoints`` as the renderer wants it: translation re-centred so that each
    superpoint rotates about its own centre (``network.py:549``)."""
    from .workloads import superpoints  # noqa: F401  (documentation pointer)
    q = sp["sp_q"].to(device)
    c = centres.to(device)
    x, y, z, w = q.unbind(-1)
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (y * w + x * z),
                     2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                     2 * (x * z - y * w), 2 * (x * w + y * z), 1 - 2 * (x * x + y * y)], dim=-1).reshape(-1, 3, 3)
    t = sp["sp_t_raw"].to(device) + c - (R @ c[..., None])[..., 0]
    return dict(sp_q=q.contiguous(), sp_t=t.contiguous(), sp_dr=sp["sp_dr"].to(device).contiguous(),
                sp_ds=sp["sp_ds"].to(device).contiguous())
