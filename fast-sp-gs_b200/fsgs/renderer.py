"""``GS_2D_fast_render`` with the reference's signature and result dictionary
(``fast_2d_gs/renderer/gs_2d_fast_render.py:670-754``) on top of ``libfsgs.so``.

Differences from routing the reference's own ``_Fast_Render`` through ``fsgs.install``:
  * the packed render records made by the preprocess kernel go straight to the compositing kernels;
  * no device-to-host read sizes the tile lists (after a device's first frame, which is sized exactly from a
    blocking read as the reference sizes every frame): they are written into a buffer whose capacity follows the
    pair count seen on earlier frames of the same size (``ListCapacity``); the counters come back asynchronously; a
    frame whose pairs did not fit comes out as NaN in every pixel (never as a plausible picture of truncated lists)
    and makes the next render call of that size on that device -- or ``check_overflow()`` -- raise;
  * optionally the superpoint LBS warp is evaluated inside the preprocess kernel (``lbs=...``).
Results are the same tensors, bit for bit, as through the operator-by-operator path.
"""
import ctypes

import torch

from . import _lib
from . import ops
from ._lib import lib, check


class ListCapacity:
    """Capacity policy for the tile lists of one device: at least ``floor`` entries, else ``growth`` x the largest
    pair count seen so far.  Counter read-backs are asynchronous (pinned buffer + event)."""

    def __init__(self, growth=1.5, floor=1 << 16):
        self.growth, self.floor = growth, floor
        self.high_water = 0
        self.last_pairs = 0  # pair count of the most recent frame whose counters have arrived
        self._pending = []  # (event, pinned counters, capacity)
        self.overflowed = 0

    def capacity(self, P, counters=None):
        """Entries to provide for the next frame.  Raises if an earlier frame overflowed (its results, and anything
        computed from them, are invalid).  Without history the pair count of this frame is read from ``counters``
        (device, written by the preprocess launch already queued): one blocking read, once per device."""
        self.check_overflow(wait=False)
        if self.high_water == 0:
            if counters is not None:
                self.high_water = int(counters[1])
                return max(self.floor, self.high_water)
            return max(self.floor, 8 * P)
        return max(self.floor, int(self.high_water * self.growth))

    def submit(self, counters, capacity):
        host = torch.empty(4, dtype=torch.int64, pin_memory=True)
        host.copy_(counters, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._pending.append((ev, host, capacity))

    def poll(self, wait=False):
        keep = []
        for ev, host, cap in self._pending:
            if wait:
                ev.synchronize()
            if ev.query():
                pairs = int(host[1])
                self.last_pairs = pairs
                self.high_water = max(self.high_water, pairs)
                if int(host[2]) > 0:
                    self.overflowed += 1
                    self.high_water = max(self.high_water, pairs)
            else:
                keep.append((ev, host, cap))
        self._pending = keep

    def check_overflow(self, wait=True):
        """Raise if an earlier frame's tile lists did not fit (that frame was rendered from truncated lists)."""
        self.poll(wait)
        if self.overflowed:
            n, self.overflowed = self.overflowed, 0
            raise RuntimeError(f"fsgs: tile lists overflowed their buffer on {n} earlier frame(s); "
                               "those frames are invalid.  The capacity has been raised; render them again.")


_capacity = {}
_last_shape = {}


def list_capacity(device=None, shape=None):
    """The capacity policy of one device and one frame shape ``(P, W, H)``: pair counts of frames of another size say
    nothing about this one.  ``shape=None`` gives the policy used last on the device (for ``check_overflow``)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if shape is None:
        shape = _last_shape.get(dev)
    _last_shape[dev] = shape
    key = (dev, shape)
    if key not in _capacity:
        _capacity[key] = ListCapacity()
    return _capacity[key]


def check_overflow(device=None):
    """Raise if any earlier frame on the device was composited from truncated lists (such frames are all NaN)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    for (d, _), cap in list(_capacity.items()):
        if d == dev:
            cap.check_overflow()


def group_pairs_by_superpoint(knn_idx, M):
    """The (Gaussian, neighbour) pairs of ``knn_idx`` [P,K] grouped by superpoint, for the atomics-free LBS adjoint:
    ``(offsets [M+1] int32, pairs [P*K] int32)`` with ``pairs`` the pair ids ``i*K + k`` in order of their superpoint.
    Built with torch ops (a sort), once per k-NN refresh; attach the result to the index tensor with
    ``knn_idx.superpoint_pairs = ...`` and the backward picks it up."""
    flat = knn_idx.reshape(-1)
    pairs = torch.argsort(flat, stable=True).to(torch.int32).contiguous()
    counts = torch.bincount(flat, minlength=M)
    offsets = torch.zeros(M + 1, dtype=torch.int32, device=knn_idx.device)
    offsets[1:] = torch.cumsum(counts, 0)
    return offsets, pairs


def make_lbs(xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds, pairs=None):
    """ctypes view of the LBS inputs (all contiguous CUDA tensors; ``knn_idx`` int64); ``pairs`` = the result of
    ``group_pairs_by_superpoint`` or None."""
    l = _lib.LBS()
    l.K, l.M = knn_idx.shape[1], sp_q.shape[0]
    for name, t in (("xyz", xyz), ("scaling_raw", scaling_raw), ("rotation_raw", rotation_raw), ("knn_idx", knn_idx),
                    ("knn_w", knn_w), ("sp_q", sp_q), ("sp_t", sp_t), ("sp_dr", sp_dr), ("sp_ds", sp_ds)):
        ops._need(t.is_cuda and t.is_contiguous(), f"lbs.{name} must be a contiguous CUDA tensor")
        setattr(l, name, t.data_ptr())
    ops._need(knn_idx.dtype == torch.int64, "lbs.knn_idx must be int64")
    if pairs is not None:
        offsets, ids = pairs
        ops._need(offsets.is_cuda and ids.is_cuda and offsets.dtype == torch.int32 and ids.dtype == torch.int32 and
                  offsets.numel() == sp_q.shape[0] + 1 and ids.numel() == knn_idx.numel(),
                  "lbs pairs: offsets [M+1] and pair ids [P*K], int32 CUDA tensors")
        l.sp_pair_offsets, l.sp_pairs = offsets.data_ptr(), ids.data_ptr()
    return l


class _LbsWarp(torch.autograd.Function):
    """Rigid LBS blend as its own operator (restates fast_2d_gs/network.py:545-573, 630-645)."""

    @staticmethod
    def forward(ctx, xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds):
        ts = [t.contiguous() for t in (xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds)]
        P = ts[0].shape[0]
        l = make_lbs(*ts)
        f32 = dict(device=xyz.device, dtype=torch.float32)
        means, scales, rots = torch.empty(P, 3, **f32), torch.empty(P, 2, **f32), torch.empty(P, 4, **f32)
        check(lib().fsgs_lbs_warp_forward(P, ctypes.byref(l), ops._ptr(means), ops._ptr(scales), ops._ptr(rots),
                                          ops._stream()), "fsgs_lbs_warp_forward")
        ctx.save_for_backward(*ts)
        ctx.pairs = getattr(knn_idx, "superpoint_pairs", None)
        return means, scales, rots

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g_means, g_scales, g_rots):
        ts = ctx.saved_tensors
        grads = lbs_backward(ts, g_means.contiguous(), g_scales.contiguous(), g_rots.contiguous(), pairs=ctx.pairs)
        return grads[0], grads[1], grads[2], None, grads[3], grads[4], grads[5], grads[6], grads[7]


def lbs_backward(ts, g_means, g_scales, g_rots, outs=(), pairs=None):
    """Gradients of the warp's eight float inputs; ``outs`` may give destinations for the first of them; ``pairs``
    (``group_pairs_by_superpoint``) selects the atomics-free superpoint reduction."""
    xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds = ts
    P = xyz.shape[0]
    l = make_lbs(*ts, pairs=pairs)
    given = list(outs) + [None] * 8
    outs = [g if g is not None else torch.empty_like(t)
            for g, t in zip(given, (xyz, scaling_raw, rotation_raw, knn_w, sp_q, sp_t, sp_dr, sp_ds))]
    g = _lib.LBSGrads()
    for name, t in zip(("g_xyz", "g_scaling_raw", "g_rotation_raw", "g_knn_w", "g_sp_q", "g_sp_t", "g_sp_dr",
                        "g_sp_ds"), outs):
        setattr(g, name, t.data_ptr())
    check(lib().fsgs_lbs_warp_backward(P, ctypes.byref(l), ops._ptr(g_means), ops._ptr(g_scales),
                                       ops._ptr(g_rots), ctypes.byref(g), ops._stream()), "fsgs_lbs_warp_backward")
    return outs


def lbs_warp(xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds):
    """-> (means [P,3], scales [P,2], rotations [P,4]) of the warped Gaussians; differentiable in every float input."""
    return _LbsWarp.apply(xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds)


class _FastRender(torch.autograd.Function):
    """preprocess -> tile binning -> compositing, and the chain of adjoints
    (the reference's ``_Fast_Render``, renderer/gs_2d_fast_render.py:592-667)."""

    @staticmethod
    def forward(ctx, means3D, scales, rotations, opacities, shs, sh_rest, Tw2v, Tv2c, Tv2s, campos, cfg, trans_mat_t2,
                culling, accum_max_count, accum_weights_p, accum_weights_count, means2D, *lbs_tensors):
        W, H, sh_degree, near_n, far_n, only_image = cfg[:6]
        use_lbs = len(lbs_tensors) == 9
        P = opacities.shape[0]
        lbs = warped = None
        if use_lbs:
            lbs_tensors = tuple(t.contiguous() for t in lbs_tensors)
            lbs = make_lbs(*lbs_tensors)
            f32 = dict(device=opacities.device, dtype=torch.float32)
            warped = (torch.empty(P, 3, **f32), torch.empty(P, 2, **f32), torch.empty(P, 4, **f32))
            means3D, scales, rotations = warped
        o = ops.preprocess_launch(W, H, sh_degree, means3D, scales, rotations, opacities, shs, sh_rest, Tw2v, Tv2s,
                                  campos, None, means2D, culling, lbs, warped)
        cap_policy = list_capacity(opacities.device, (P, W, H))
        capacity = cap_policy.capacity(P, o["counters"])
        ranges, point_list, tile_order = ops.bin_launch(W, H, o, opacities, capacity)
        cap_policy.submit(o["counters"], capacity)
        outs = ops.render_forward_launch(W, H, near_n, far_n, only_image, P, o["records"], point_list, ranges,
                                         tile_order, trans_mat_t2, accum_max_count, accum_weights_p,
                                         accum_weights_count, counters=o["counters"])
        pixel_colors, pixel_opacity, pixel_extras, pixel_flow, n_contrib = outs
        ctx.cfg = cfg
        ctx.lbs_pairs = getattr(lbs_tensors[3], "superpoint_pairs", None) if use_lbs else None
        ctx.set_materialize_grads(False)  # outputs without an upstream gradient arrive as None, not as zeros
        ctx.use_lbs = use_lbs
        ctx.has = (sh_rest is not None, trans_mat_t2 is not None, pixel_extras is not None, pixel_flow is not None)
        saved = [means3D, scales, rotations, opacities, shs, Tw2v, Tv2s, campos, o["means2D"], o["trans_mat"],
                 o["radii"], o["colors"], o["records"], ranges, point_list, tile_order, pixel_opacity, n_contrib]
        saved += [t for t in (sh_rest, trans_mat_t2, pixel_extras, pixel_flow) if t is not None]
        saved += list(lbs_tensors) if use_lbs else []
        ctx.save_for_backward(*saved)
        ctx.mark_non_differentiable(n_contrib, o["radii"])
        return pixel_colors, pixel_opacity, pixel_extras, pixel_flow, n_contrib, o["radii"]

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g_colors, g_opacity, g_extras, g_flow, _g_nc, _g_radii):
        W, H, sh_degree, near_n, far_n, only_image = ctx.cfg[:6]
        grad_out = (ctx.cfg[6] if len(ctx.cfg) > 6 else None) or {}

        def dest(name, like):
            """A fresh alias of the caller's destination for this gradient (autograd can then adopt it as ``.grad``
            without a copy), or None."""
            t = grad_out.get(name)
            if t is None or like is None:
                return None
            ops._need(t.is_cuda and t.is_contiguous() and t.dtype == torch.float32 and t.shape == like.shape,
                      f"grad_out[{name!r}] must be a contiguous float32 CUDA tensor of shape {tuple(like.shape)}")
            return t.detach()

        sv = list(ctx.saved_tensors)
        (means3D, scales, rotations, opacities, shs, Tw2v, Tv2s, campos, means2D, trans_mat, radii, colors, records,
         ranges, point_list, tile_order, pixel_opacity, n_contrib) = sv[:18]
        rest = sv[18:]
        has_rest, has_t2, has_extras, has_flow = ctx.has
        sh_rest = rest.pop(0) if has_rest else None
        trans_mat_t2 = rest.pop(0) if has_t2 else None
        pixel_extras = rest.pop(0) if has_extras else None
        rest.pop(0) if has_flow else None
        lbs_tensors = rest if ctx.use_lbs else None
        P = opacities.shape[0]
        dev = opacities.device
        zeros = lambda *s: torch.zeros(*s, device=dev, dtype=torch.float32)
        g_colors = g_colors.contiguous() if g_colors is not None else zeros(3, H, W)
        g_opacity = g_opacity.contiguous() if g_opacity is not None else zeros(H, W)
        # no upstream gradient on the auxiliary channels (a loss on image and opacity only): the backward kernel
        # then skips their terms and reduces 15 instead of 21 components per splat
        aux = has_extras and (g_extras is not None or (has_flow and g_flow is not None))
        if aux and g_extras is None:
            g_extras = zeros(8, H, W)
        flow = aux and has_flow and g_flow is not None
        g_col, g_m2d, g_tm, g_im, g_no = ops.render_backward_launch(
            W, H, near_n, far_n, P, records, point_list, ranges, tile_order, trans_mat_t2 if flow else None,
            pixel_opacity, pixel_extras if aux else None, n_contrib, g_colors, g_opacity,
            g_extras.contiguous() if aux else None, g_flow.contiguous() if flow else None)
        # one block for all parameter gradients; the kernel writes every row (zeros for culled Gaussians)
        n_sh = shs.numel() // max(P, 1)
        n_rest = sh_rest.numel() // max(P, 1) if has_rest else 0
        want_sh = sh_degree >= 0
        gsh = dest("sh_features", shs) if want_sh else None
        grest = dest("sh_features_rest", sh_rest) if (want_sh and has_rest) else None
        width = 3 + 2 + 4 + 1 + (n_sh if want_sh and gsh is None else 0) + (n_rest if want_sh and grest is None else 0)
        Pp = (P + 63) & ~63  # every view starts on a 256-byte boundary: the kernels store float2 / float4 rows
        block = torch.empty(Pp * width, device=dev, dtype=torch.float32)
        off = 0

        def take(n, shape):
            nonlocal off
            v = block[off * Pp:off * Pp + n * P].view(shape)
            off += n
            return v

        gm, gs, gr, go = take(3, (P, 3)), take(2, (P, 2)), take(4, (P, 4)), take(1, (P, 1))
        if want_sh and gsh is None:
            gsh = take(n_sh, shs.shape)
        if want_sh and has_rest and grest is None:
            grest = take(n_rest, sh_rest.shape)
        a = _lib.PreprocessBwdArgs()
        a.P, a.W, a.H, a.sh_degree = P, W, H, sh_degree
        a.n_dc = shs.shape[1] if sh_degree >= 0 else 1
        a.n_rest = sh_rest.shape[1] if has_rest else 0
        p = ops._ptr
        a.means, a.scales, a.rots, a.shs, a.sh_rest = p(means3D), p(scales), p(rotations), p(shs), p(sh_rest)
        a.Tw2v, a.Tv2s, a.campos, a.trans_mat, a.colors, a.radii = p(Tw2v), p(Tv2s), p(campos), p(trans_mat), p(colors), p(radii)
        a.grad_means2D, a.grad_trans_mat, a.grad_inverse_m = p(g_m2d), p(g_tm), p(g_im)
        a.grad_colors, a.grad_normal_opacity = p(g_col), p(g_no)
        a.grad_means, a.grad_scales, a.grad_rots, a.grad_opac = p(gm), p(gs), p(gr), p(go)
        a.grad_shs, a.grad_sh_rest = p(gsh), p(grest)
        check(lib().fsgs_preprocess_backward(ctypes.byref(a), ops._stream()), "fsgs_preprocess_backward")
        if grad_out.get("on_sh_ready") is not None:
            grad_out["on_sh_ready"]()  # the SH gradients are final in stream order: their exchange may start
        if sh_degree < 0:
            gsh = g_col  # colours were an input: their gradient is the compositing gradient itself
        grads = [gm, gs, gr, go, gsh, grest, None, None, None, None, None, None, None, None, None, None, g_m2d]
        if ctx.use_lbs:
            lg = lbs_backward(lbs_tensors, gm, gs, gr, pairs=ctx.lbs_pairs,
                              outs=(dest("xyz", lbs_tensors[0]), dest("scaling_raw", lbs_tensors[1]),
                                    dest("rotation_raw", lbs_tensors[2])))
            grads[0] = grads[1] = grads[2] = None
            grads += [lg[0], lg[1], lg[2], None, lg[3], lg[4], lg[5], lg[6], lg[7]]
        return tuple(grads)


_pixel_grid = {}


def _homogeneous_pixels(W, H, device):
    """[H*W, 3] rows (x, y, 1), cached per image size and device."""
    key = (W, H, str(device))
    if key not in _pixel_grid:
        gx, gy = torch.meshgrid(torch.arange(W, device=device).float(), torch.arange(H, device=device).float(),
                                indexing="xy")
        _pixel_grid[key] = torch.stack([gx, gy, torch.ones_like(gx)], dim=-1).reshape(-1, 3).contiguous()
    return _pixel_grid[key]


def depths_to_points(Tw2v, Tv2c, size, depthmap):
    """Back-project a depth map to world points (renderer/gs_2d_fast_render.py:558-575).  Same arithmetic, but
    device-agnostic, without the error-checking (synchronising) matrix inverses, with the pixel grid cached and the
    two 3x3 factors multiplied together before they meet the [H*W,3] pixel matrix."""
    c2w = torch.linalg.inv_ex(Tw2v).inverse
    W, H = size
    ndc2pix = torch.tensor([[W / 2, 0, 0, W / 2], [0, H / 2, 0, H / 2], [0, 0, 0, 1]], dtype=torch.float32,
                           device=Tw2v.device).T
    projection_matrix = c2w.T @ (Tv2c @ Tw2v).T
    intrins = (projection_matrix @ ndc2pix)[:3, :3].T
    rays_d = _homogeneous_pixels(W, H, Tw2v.device) @ (torch.linalg.inv_ex(intrins).inverse.T @ c2w[:3, :3].T)
    return depthmap.reshape(-1, 1) * rays_d + c2w[:3, 3]


def depth_to_normal(Tw2v, Tv2c, size, depth):
    """Pseudo surface normal from a depth map (renderer/gs_2d_fast_render.py:578-589)."""
    points = depths_to_points(Tw2v, Tv2c, size, depth).reshape(*depth.shape[1:], 3)
    output = torch.zeros_like(points)
    dx = points[2:, 1:-1] - points[:-2, 1:-1]
    dy = points[1:-1, 2:] - points[1:-1, :-2]
    output[1:-1, 1:-1, :] = torch.nn.functional.normalize(torch.linalg.cross(dx, dy, dim=-1), dim=-1)
    return output


class _SurfaceEpilogue(torch.autograd.Function):
    """normals to world space, surface depth, pseudo surface normal: one kernel forward, one backward."""

    @staticmethod
    def forward(ctx, out_extras, opacities, Tw2v, Tv2c, depth_ratio):
        _, H, W = out_extras.shape
        f32 = dict(device=out_extras.device, dtype=torch.float32)
        normals, surf_depth, surf_normal = torch.empty(3, H, W, **f32), torch.empty(1, H, W, **f32), torch.empty(3, H, W, **f32)
        p = ops._ptr
        check(lib().fsgs_epilogue_forward(W, H, float(depth_ratio), p(Tw2v), p(Tv2c), p(out_extras), p(opacities),
                                          p(normals), p(surf_depth), p(surf_normal), ops._stream()),
              "fsgs_epilogue_forward")
        ctx.save_for_backward(out_extras, opacities, Tw2v, Tv2c)
        ctx.ratio = float(depth_ratio)
        return normals, surf_depth, surf_normal

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g_normals, g_depth, g_surf_normal):
        out_extras, opacities, Tw2v, Tv2c = ctx.saved_tensors
        _, H, W = out_extras.shape
        g_extras = torch.empty_like(out_extras)
        p = ops._ptr
        c = lambda t: None if t is None else t.contiguous()
        g_normals, g_depth, g_surf_normal = c(g_normals), c(g_depth), c(g_surf_normal)
        check(lib().fsgs_epilogue_backward(W, H, ctx.ratio, p(Tw2v), p(Tv2c), p(out_extras), p(opacities),
                                           p(g_normals), p(g_depth), p(g_surf_normal), p(g_extras), ops._stream()),
              "fsgs_epilogue_backward")
        return g_extras, None, None, None, None


def GS_2D_fast_render(points, scales, rotations, opacity, size, Tw2v, Tv2c, Tv2s, campos=None, focals=None, FoV=None,
                      is_opengl=False, near=0.2, far=100, sh_degree=0, colors=None, sh_features=None,
                      sh_features_rest=None, depth_ratio=1., culling=None, accum_max_count=None,
                      accum_weights_p=None, accum_weights_count=None, trans_mat_t2=None, lbs=None, only_image=False,
                      grad_out=None, **kwargs):
    """Render one view.  Same arguments and result dictionary as the reference's ``GS_2D_fast_render``
    (renderer/gs_2d_fast_render.py:670-754): ``images [3,H,W]``, ``normals`` (world space), ``opacity``,
    ``distortion``, ``surf_depth``, ``surf_normal``, ``radii``, ``viewspace_points`` (its ``.grad`` receives the
    densification proxy), ``visibility_filter``, ``flows``.  No background is composited.

    Extra, optional: ``lbs=(xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds)`` evaluates the
    superpoint warp inside the preprocess kernel (then ``points/scales/rotations`` are ignored);
    ``only_image=True`` skips the auxiliary channels and returns only images / opacity / radii entries;
    ``grad_out={name: tensor}`` (names ``sh_features``, ``sh_features_rest`` and, with ``lbs``, ``xyz``,
    ``scaling_raw``, ``rotation_raw``) makes the backward kernels write those gradients straight into the caller's
    tensors (slices of a communication bucket, say) instead of fresh allocations; the tensors returned to autograd
    alias them.  Only valid while the corresponding leaves have no ``.grad`` yet.  An entry ``on_sh_ready`` (a
    callable) is invoked in the backward as soon as the SH gradients have been queued, before the LBS adjoint.
    """
    P = opacity.shape[0]
    means2D = torch.zeros(P, 2, device=opacity.device, dtype=torch.float32, requires_grad=True)
    W, H = (int(v) for v in size)
    if campos is None:
        campos = torch.linalg.inv_ex(Tw2v).inverse[:3, 3].contiguous()
    feats = sh_features if colors is None else colors
    cfg = (W, H, int(sh_degree) if colors is None else -1, float(near), float(far), bool(only_image), grad_out)
    geom = (points, scales, rotations)
    if lbs is None:
        geom = tuple(t.contiguous() for t in geom)
    lbs_args = tuple(lbs) if lbs is not None else ()
    images, opacities, out_extras, flows, n_contrib, radii = _FastRender.apply(
        geom[0], geom[1], geom[2], opacity.contiguous(), feats.contiguous(),
        None if sh_features_rest is None or colors is not None else sh_features_rest.contiguous(),
        Tw2v.contiguous(), Tv2c.contiguous(), Tv2s.contiguous(), campos.contiguous(), cfg, trans_mat_t2, culling,
        accum_max_count, accum_weights_p, accum_weights_count, means2D, *lbs_args)
    out = {"images": images, "opacity": opacities, "radii": radii, "viewspace_points": means2D,
           "visibility_filter": radii > 0, "flows": flows}
    if only_image:
        return out
    Tw2v_c, Tv2c_c = Tw2v.contiguous(), Tv2c.contiguous()
    normals, surf_depth, surf_normal = _SurfaceEpilogue.apply(out_extras, opacities.detach(), Tw2v_c, Tv2c_c,
                                                              depth_ratio)
    distortion = out_extras[5:6]
    out.update(normals=normals, distortion=distortion, surf_depth=surf_depth, surf_normal=surf_normal)
    return out
