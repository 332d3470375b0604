"""A minimal dynamic surfel scene: the parameters the reference model owns (``fast_2d_gs/network.py:357``:
positions, 2 log-scales, rotation, opacity logit, SH DC + 15 rest coefficients = 58 floats per Gaussian), the
superpoint k-NN / LBS weights (``network.py:498-521``, 'dist' weighting) and one training step
(warp -> render -> backward -> visibility-masked Adam) as ``train.py:343-412`` runs it; the upstream image
gradient is an input or comes from the fused L1 + SSIM loss.  Training runs on ``fsgs.engine.ViewEngine`` (two C
calls per view, gradients of several views summed in place, one exchange per step); ``render`` is the autograd
operator ``GS_2D_fast_render`` for everything else.
"""
import torch
import torch.distributed as dist

from . import ops
from .dist import GradBucket, slot_order
from .optim import DenseAdam, SparseGaussianAdam
from .renderer import GS_2D_fast_render, check_overflow, group_pairs_by_superpoint

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
    def __init__(self, surfels, centres, K=3, eps=1e-15, device="cuda", lrs=None, motion_net=None, kernel_weights=None,
                 lr_deform=1.6e-4):
        """``motion_net``: a ``fsgs.motion.MotionNet``; views may then give a time ``t`` instead of a precomputed
        ``motion`` and the network is trained with the scene.  ``kernel_weights``: ``(raw_radius [M], raw_weight [M] or
        None)`` switches the LBS weights to the learnable kernel form of the shipped configuration
        (network.py:506-513), re-evaluated every step and trained as well.  Both are optimised by a dense Adam at
        ``lr_deform`` (the reference's deformation-network group, network.py:296-305)."""
        P = lambda t: torch.nn.Parameter(t.to(device).contiguous())
        self.xyz = P(surfels["means"])
        self.scaling = P(surfels["log_scales"])
        self.rotation = P(surfels["rots_raw"])
        self.opacity = P(surfels["opac_raw"])
        self.sh_dc = P(surfels["sh_dc"])
        self.sh_rest = P(surfels["sh_rest"])
        self.centres = centres.to(device).contiguous()
        self.K = K
        self.motion_net = motion_net
        self.sp_radius = self.sp_weight = None
        if kernel_weights is not None:
            self.sp_radius = P(kernel_weights[0])
            self.sp_weight = P(kernel_weights[1]) if kernel_weights[1] is not None else None
        self.dense_params = ([motion_net.params] if motion_net is not None else []) + \
            [p for p in (self.sp_radius, self.sp_weight) if p is not None]
        self.dense_optimizer = DenseAdam(self.dense_params, lr=lr_deform, eps=eps) if self.dense_params else None
        self.refresh_knn()
        LRS = dict(globals()["LRS"], **(lrs or {}))
        groups = [dict(params=[self.xyz], lr=LRS["xyz"]), dict(params=[self.sh_dc], lr=LRS["sh_dc"]),
                  dict(params=[self.sh_rest], lr=LRS["sh_rest"]), dict(params=[self.opacity], lr=LRS["opacity"]),
                  dict(params=[self.scaling], lr=LRS["scaling"]), dict(params=[self.rotation], lr=LRS["rotation"])]
        self.optimizer = SparseGaussianAdam(groups, lr=0.0, eps=eps)
        self.bucket = None
        self.engine = None
        self.sh_send = self.sh_recv = None   # SH-gradient factors of the views: this rank's slots, everybody's
        self.trace = None                    # a list: train_views appends (label, CUDA event) at its phase boundaries
        self.track_densification = False

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
        self.knn_idx, self.knn_d2 = idx, d2
        if self.sp_radius is not None:
            from .motion import kernel_weights
            self.knn_w = kernel_weights(d2, idx, self.sp_radius.data, None if self.sp_weight is None else self.sp_weight.data)
        else:
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

    # ---- training ---------------------------------------------------------------------------------------------
    def _engine(self, size):
        from .engine import ViewEngine
        W, H = (int(v) for v in size)
        e = self.engine
        if e is None or (e.W, e.H, e.P) != (W, H, self.num_points):
            e = self.engine = ViewEngine(self.num_points, W, H, self.K, self.centres.shape[0], self.xyz.device)
        return e

    def _grad_bucket(self):
        """One flat buffer for all leaf gradients and the visibility mask (as floats): the backward kernels write and
        accumulate straight into it, and it is what the ranks exchange.  Segments: SH DC, SH rest, mask | position,
        opacity, scale, rotation -- the first three are final as soon as the preprocess adjoint has run."""
        if self.bucket is None:
            self.bucket = GradBucket([self.sh_dc, self.sh_rest, self.xyz, self.opacity, self.scaling, self.rotation] +
                                     self.dense_params, extra=self.num_points, extra_after=1)
            self.g_knn_w = torch.zeros_like(self.knn_w)
            M = self.centres.shape[0]
            z = lambda k: torch.zeros(M, k, device=self.xyz.device)
            self.motion_grads = dict(sp_q=z(4), sp_t=z(3), sp_dr=z(4), sp_ds=z(2))
            self.motion_buf = dict(sp_q=z(4), sp_t=z(3), sp_dr=z(4), sp_ds=z(2))
        return self.bucket

    def train_views(self, views, size, group=None, distributed=False, views_per_rank=None, exchange="factors"):
        """One iteration over the views this rank owns: for each view forward and backward (``libfsgs`` launches only,
        two C calls per view), the per-Gaussian gradients of the views summed in place in call order; then -- when
        ``distributed`` -- ONE exchange with the other ranks; then the fused visibility-masked Adam.  The reference's
        serial loop over a batch of views, ``fast_2d_gs/network.py:683-745``, followed by ``train.py:402-405``.

        The exchange.  48 of the 59 gradient floats of a Gaussian are SH coefficients, and a view's SH gradient is an
        outer product: (clamped colour gradient, 3 floats) x (SH basis of the view direction, a function of 3 floats).
        ``exchange="factors"`` therefore all-gathers those six floats per Gaussian and view, with the view's visibility
        as a seventh (started after the last view's compositing adjoint, under its preprocess and LBS adjoints),
        all-reduces the remaining ten floats (plus the dense parameters' gradients) after the LBS adjoint, and rebuilds
        the summed SH gradient and the summed mask on every rank in view order (``ops.sh_grad_from_views``): every rank
        forms the same bits, the replicas stay identical, and 7 V floats per Gaussian travel instead of 49 through an
        all-reduce.  ``views_per_rank``: the number of view slots every rank contributes -- the same on all ranks;
        default ``max(len(views), 1)``, to be passed explicitly when ranks hold different numbers of views.
        ``exchange="rows"`` all-reduces the gradient rows themselves (two all-reduces: SH and mask first, the rest
        behind).  ``self.trace``: set it to a list and the phase boundaries are appended as (label, CUDA event).

        ``views``: list of dicts with ``cam`` (``Tw2v, Tv2s, campos``), ``motion`` (``sp_q, sp_t, sp_dr, sp_ds``) -- or,
        with a motion network, ``t`` (float32 CUDA tensor with one element: the motion is then evaluated by the network
        and the network is trained; all views of a step must use the same form) --,
        ``g_images`` -- a [3,H,W] tensor, or a callable ``engine -> [3,H,W]`` evaluated after the view's forward (a
        loss) --, and optionally ``g_opacity [H,W]``, ``g_extras [8,H,W]``, ``on_motion_grads`` (a callable run after the
        view's backward has been queued, while ``self.motion_grads`` hold this view's superpoint-motion gradients).
        Returns the engine, whose ``images / opacity / extras / radii`` are those of the last view."""
        eng, b = self._engine(size), self._grad_bucket()

        def mark(label):
            if self.trace is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self.trace.append((label, ev))

        mark("start")
        world = dist.get_world_size(group) if distributed and dist.is_available() and dist.is_initialized() else 1
        factors = distributed and world > 1 and exchange == "factors" and eng.sh_degree <= 3
        n_slots = max(len(views), 1) if views_per_rank is None else int(views_per_rank)
        if factors and len(views) > n_slots:
            raise ValueError("more views than views_per_rank")
        dst = dict(xyz=b.view_of(self.xyz), scaling=b.view_of(self.scaling), rotation=b.view_of(self.rotation),
                   opacity=b.view_of(self.opacity), sh_dc=None if factors else b.view_of(self.sh_dc),
                   sh_rest=None if factors else b.view_of(self.sh_rest),
                   visible=None if factors else b.extra,   # factors: every view's visibility rides in its slot
                   knn_w=self.g_knn_w, **self.motion_grads)
        if factors:
            P = self.num_points
            F = ops.SH_SOURCE_FLOATS
            if self.sh_send is None or tuple(self.sh_send.shape) != (n_slots, P, F) or self.sh_recv.shape[0] != world * n_slots:
                self.sh_send = torch.zeros(n_slots, P, F, device=self.xyz.device)
                self.sh_recv = torch.empty(world * n_slots, P, F, device=self.xyz.device)
            if len(views) < n_slots:
                self.sh_send[len(views):].zero_()   # slots without a view add nothing
        early = late = gather = None
        last_seg = len(b.bounds) - 1
        net, n_timed = self.motion_net, 0
        if self.sp_radius is not None:  # the kernel weights follow their parameters: one launch per step
            from .motion import kernel_weights
            kernel_weights(self.knn_d2, self.knn_idx, self.sp_radius.data,
                           None if self.sp_weight is None else self.sp_weight.data, out=self.knn_w)

        def after_view(v):
            nonlocal n_timed
            if self.track_densification:
                ops.densify_stats(eng.viewspace_grad, eng.radii, self.grad_accum, self.grad_denom, self.max_radii)
            if "t" in v:  # this view's motion gradients -> network parameters, summed over the views
                net.backward(self.motion_grads, b.view_of(net.params), accumulate=n_timed > 0)
                n_timed += 1
            if v.get("on_motion_grads") is not None:
                v["on_motion_grads"](self.motion_grads)

        def after_last_view():
            if self.sp_radius is not None:
                from .motion import kernel_weights_backward
                kernel_weights_backward(self.knn_d2, self.knn_idx, self.sp_radius.data,
                                        None if self.sp_weight is None else self.sp_weight.data, self.g_knn_w,
                                        self.knn_idx.superpoint_pairs, b.view_of(self.sp_radius),
                                        None if self.sp_weight is None else b.view_of(self.sp_weight))

        def first_exchange():
            """What is final by now leaves while the rest of the last view's backward runs."""
            nonlocal early, gather
            if factors:
                gather = dist.all_gather_into_tensor(self.sh_recv.view(-1), self.sh_send.view(-1), group=group, async_op=True)
            else:
                early = b.reduce_span(0, 2, group)   # SH gradients and the mask

        for j, v in enumerate(views):
            motion = net.forward(self.centres, v["t"], out=self.motion_buf) if "t" in v else v["motion"]
            eng.forward(self, v["cam"], motion)
            g_images = v["g_images"]
            if callable(g_images):
                g_images = g_images(eng)
            args = (g_images, v.get("g_opacity"), v.get("g_extras"), dst)
            src = self.sh_send[j] if factors else None
            if distributed and j == len(views) - 1:
                # factors: they and the mask are known once the compositing adjoint has run (phase 3), and travel
                # under the preprocess and LBS adjoints (phase 4); rows: the SH rows need the preprocess adjoint
                # (phase 1) and travel under the LBS adjoint (phase 2)
                eng.backward(*args, accumulate=j > 0, phase=3 if factors else 1, sh_source=src)
                mark("first part of the last backward")
                first_exchange()
                eng.backward(*args, accumulate=j > 0, phase=4 if factors else 2, sh_source=src)
                after_view(v)
                after_last_view()
                mark("rest of the last backward")
                late = b.reduce_span(3, last_seg, group)
            else:
                eng.backward(*args, accumulate=j > 0, sh_source=src)
                after_view(v)
                if j == len(views) - 1:
                    after_last_view()
        if not views:  # a rank without a view this step still takes part in the exchange, with zeros
            b.flat.zero_()
            if distributed:
                first_exchange()
                late = b.reduce_span(3, last_seg, group)
        elif net is not None and n_timed == 0:
            b.view_of(net.params).zero_()
        b.adopt()
        self.optimizer.set_before_step(b.extra, self.num_points)  # float mask: visible where > 0
        if gather is not None:
            gather.wait()
            mark("all-gather arrived")
            # summed in view order on every rank
            ops.sh_grad_from_views(self.sh_recv, slot_order(world, n_slots), eng.sh_degree, b.view_of(self.sh_dc),
                                   b.view_of(self.sh_rest), visible=b.extra)
            mark("SH rows and mask rebuilt")
        if early is not None:
            early.wait()
            mark("first all-reduce arrived")
        self.optimizer.step_visible(only=[self.sh_dc, self.sh_rest])
        mark("SH Adam")
        if late is not None:
            late.wait()
            mark("last all-reduce arrived")
        self.optimizer.step_visible(only=[self.xyz, self.opacity, self.scaling, self.rotation])
        mark("rest of Adam")
        if self.dense_optimizer is not None:
            # a view whose tile lists overflowed (on any rank) left -inf in the mask: the masked Adam above passed no
            # row, and the dense parameters' Adam is gated by the same element (mask values are >= 0 otherwise)
            self.dense_optimizer.step_gated(b.extra[:1] + 1.0)
        self._drop_grads()
        return eng

    def last_step_dropped(self):
        """True when the last ``train_views`` step was dropped on the device because a view's tile lists overflowed
        their buffer on some rank (one scalar read: synchronises).  The same on every rank."""
        return self.bucket is not None and bool(torch.isinf(self.bucket.extra[0]))

    def train_step(self, cam, size, motion, g_images, g_opacity, group=None, distributed=False, g_aux=None):
        """One iteration on one view with the given upstream gradients on images [3,H,W] and opacity [H,W] (and, with
        ``g_aux = {"normals": [3,H,W] (world space), "distortion": [1,H,W], "surf_depth": ..., "surf_normal": ...}``,
        on those entries of the render dictionary).  Returns a dictionary with the view's ``images``, ``opacity``,
        ``extras``, ``radii`` and ``visibility_filter`` (buffers of the engine: valid until the next view)."""
        view = dict(cam=cam, motion=motion, g_images=g_images, g_opacity=g_opacity)
        if g_aux:
            def with_aux(eng):  # the auxiliary gradient needs the forward's extras: both are evaluated after the forward
                view["g_extras"] = self._extras_gradient(eng, cam, g_aux)
                return g_images(eng) if callable(g_images) else g_images
            view["g_images"] = with_aux
        eng = self.train_views([view], size, group=group, distributed=distributed)
        return dict(images=eng.images, opacity=eng.opacity, extras=eng.extras, radii=eng.radii,
                    visibility_filter=eng.radii > 0)

    def _extras_gradient(self, eng, cam, g_aux, depth_ratio=1.0):
        """Upstream gradients on the entries of the render dictionary derived from the auxiliary channels -> the
        gradient of the [8,H,W] channels themselves (adjoint of the epilogue kernel; distortion is channel 5)."""
        from ._lib import check, lib
        p = ops._ptr
        g_extras = torch.empty_like(eng.extras)
        c = lambda t: None if t is None else t.contiguous()
        check(lib().fsgs_epilogue_backward(eng.W, eng.H, float(depth_ratio), p(cam["Tw2v"].contiguous()),
                                           p(cam["Tv2c"].contiguous()), p(eng.extras), p(eng.opacity),
                                           p(c(g_aux.get("normals"))), p(c(g_aux.get("surf_depth"))),
                                           p(c(g_aux.get("surf_normal"))), p(g_extras), ops._stream()),
              "fsgs_epilogue_backward")
        if g_aux.get("distortion") is not None:
            g_extras[5:6] += g_aux["distortion"]
        return g_extras

    def train_step_with_loss(self, cam, size, motion, target, lambda_l1=0.8, lambda_ssim=0.2, group=None,
                             distributed=False):
        """One iteration against a target image [3,H,W]: forward, fused L1 + SSIM loss and its image gradient
        (``fsgs.loss``), backward, optimiser.  Returns (render dictionary, loss as a device scalar)."""
        from .loss import l1_ssim_value_and_grad
        holder = {}

        def upstream(eng):
            holder["loss"], g = l1_ssim_value_and_grad(eng.images, target, lambda_l1, lambda_ssim)
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
        extra = [self.knn_idx, self.knn_w, self.knn_d2]
        if self.track_densification:
            extra += [self.grad_accum, self.grad_denom, self.max_radii]
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
        self.knn_idx, self.knn_w, self.knn_d2 = rest[:3]
        if self.track_densification:
            self.grad_accum, self.grad_denom, self.max_radii = rest[3:6]
        self.knn_idx.superpoint_pairs = group_pairs_by_superpoint(self.knn_idx, self.centres.shape[0])
        self.bucket = None
        self.engine = None
        return self.num_points

    @torch.no_grad()
    def densify(self, max_grad, extent, percent_dense=0.01, N=2, noise=None, generator=None):
        """Clone the small and split the large Gaussians whose mean screen-space gradient reached ``max_grad``
        (``densify``, fast_2d_gs/gaussian_splatting.py:623-628, with the 2-D split of network.py:1156-1185): selection,
        the split children's positions and scales, and the move of all six parameters and twelve Adam moments into
        their new rows (kept originals, clones, children copy 0 .. N-1; fresh moments zero) run on the device in four
        launches.  ``noise`` [n_split * N, 2]: the standard-normal draws to use (else drawn from ``generator``).
        Needs ``track_densification`` to have gathered statistics.  Returns (n_clone, n_split)."""
        P = self.num_points
        flags = ops.densify_select(self.grad_accum, self.grad_denom, self.scaling.data, max_grad, percent_dense * extent)
        idx = torch.arange(P, device=flags.device, dtype=torch.int32)
        keep, clone, split = idx[flags != 2], idx[flags == 1], idx[flags == 2]   # sizes read back: one sync each
        n_keep, n_clone, n_split = keep.numel(), clone.numel(), split.numel()
        parents = split.repeat(N)
        index = torch.cat([keep, clone, parents])
        fresh = torch.full((n_clone + N * n_split,), -1, dtype=torch.int32, device=flags.device)
        params = self.params
        moments = []
        for p in params:
            st = self.optimizer.state.get(p, {})
            moments += [st.get("exp_avg"), st.get("exp_avg_sq")]
        have = [m for m in moments if m is not None]
        new_params = ops.gather_rows([p.data for p in params], index)
        new_moments = ops.gather_rows(have, torch.cat([keep, fresh])) if have else []
        if n_split:
            if noise is None:
                noise = torch.randn(N * n_split, 2, device=flags.device, generator=generator)
            names = [id(p) for p in params]
            x_new, s_new = new_params[names.index(id(self.xyz))], new_params[names.index(id(self.scaling))]
            ops.split_children(parents, noise.contiguous(), self.xyz.data, self.scaling.data, self.rotation.data, N,
                               x_new[n_keep + n_clone:], s_new[n_keep + n_clone:])
        self._install(params, [torch.nn.Parameter(t) for t in new_params], new_moments)
        self.refresh_knn()   # the new Gaussians need neighbours
        return n_clone, n_split

    def _install(self, old_params, new_params, new_moments):
        """Swap in resized parameter tensors and their Adam moments (``change_optimizer``, gaussian_splatting.py:498-548)
        and reset everything that is sized by the Gaussian count."""
        new_moments = list(new_moments)
        for group, old, new in zip(self.optimizer.param_groups, old_params, new_params):
            st = self.optimizer.state.pop(old, None)
            group["params"][0] = new
            if st:
                st["exp_avg"], st["exp_avg_sq"] = new_moments.pop(0), new_moments.pop(0)
                self.optimizer.state[new] = st
        self.xyz, self.sh_dc, self.sh_rest, self.opacity, self.scaling, self.rotation = new_params
        self.bucket = None
        self.engine = None
        if self.track_densification:
            self.track_densification = False
            self.enable_densification_stats()

    def enable_densification_stats(self):
        """Start (or restart, zeroed) gathering the statistics ``densify`` selects by: per Gaussian the summed norm of
        the screen-space gradient, the number of views it was visible in, and its largest radius
        (``add_densification_stats``, network.py:1143-1154); updated by one small launch per training view."""
        z = lambda: torch.zeros(self.num_points, device=self.xyz.device)
        self.grad_accum, self.grad_denom, self.max_radii = z(), z(), z()
        self.track_densification = True

    def _drop_grads(self):
        for p in self.params + self.dense_params:  # zero_grad(set_to_none=True) without the optimizer's hook layers
            p.grad = None

    def check(self):
        """Raise if a tile list overflowed on an earlier view (``render`` path or training views)."""
        check_overflow(self.xyz.device)
        if self.engine is not None:
            self.engine.check()


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
