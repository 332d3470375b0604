"""The reference's operator names over ``libfsgs.so``.

Each callable below has the name, positional arguments, return values and in-place behaviour of the
pybind11 function of the same name in the reference extension ``fast_2d_gs/_C`` (sources under
``fast_2d_gs/_C/src``; the line numbers are given per operator).  Tensors are allocated with torch, raw
pointers and the current CUDA stream go to the C ABI.  Errors surface as ``RuntimeError`` like the
reference's ``TORCH_CHECK``s.  There is no CPU path.
"""
import ctypes

import torch

from . import _lib
from ._lib import lib, check

TILE = 16
REC = 32  # floats per packed render record


class _Op:
    """A plain callable that does not bind as a method when stored on a class (pybind functions behave the same;
    ``SparseGaussianAdam._update_C`` relies on it)."""

    def __init__(self, fn):
        self._fn = fn
        self.__name__ = fn.__name__
        self.__doc__ = fn.__doc__

    def __call__(self, *args, **kwargs):
        return self._fn(*args, **kwargs)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """Handle of torch's current stream on the current device (the raw getter costs a fraction of a microsecond; the
    Stream object route costs several, ten times per frame)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _check_input(t, name, shape=None, dtype=torch.float32):
    _need(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.dtype == dtype, f"{name} must be a {dtype} tensor")
    if shape is not None:
        _need(tuple(t.shape) == tuple(shape), f"{name} have error shape")


def _tiles(W, H):
    return (W + TILE - 1) // TILE, (H + TILE - 1) // TILE


class RenderAux:
    """What the compositing kernels want beyond the reference's tensors: packed records and the tile launch order.
    Travels as an attribute of ``point_list`` so that a preprocess -> render -> backward chain packs only once."""
    __slots__ = ("records", "tile_order", "versions")

    def __init__(self, records, tile_order, tensors):
        self.records, self.tile_order = records, tile_order
        self.versions = tuple((t.data_ptr(), t._version) for t in tensors)

    def matches(self, tensors):
        return self.versions == tuple((t.data_ptr(), t._version) for t in tensors)


def _alloc_preprocess_outputs(P, T, dev, sh_degree, shs, means2D, trans_precomp, want_records=True):
    f32 = dict(device=dev, dtype=torch.float32)
    out = {
        "means2D": means2D if means2D is not None else torch.empty(P, 2, **f32),
        "colors": shs if sh_degree < 0 else torch.empty(P, 3, **f32),
        "trans_mat": trans_precomp if trans_precomp is not None else torch.empty(P, 3, 3, **f32),
        "inverse_m": torch.empty(P, 3, 3, **f32),
        "normal_opacity": torch.empty(P, 4, **f32),
        "depths": torch.empty(P, **f32),
        "radii": torch.empty(P, device=dev, dtype=torch.int32),
        "tiles_touched": torch.empty(P, device=dev, dtype=torch.int32),
        "records": torch.empty(P, REC, **f32) if want_records else None,
        "tile_counts": torch.empty(T, device=dev, dtype=torch.int32),
        "counters": torch.empty(_lib_num_counters(), device=dev, dtype=torch.int64),
    }
    return out


def _lib_num_counters():
    return 4


def preprocess_launch(W, H, sh_degree, means3D, scales, rotations, opacities, shs, sh_rest, Tw2v, Tv2s, campos,
                      trans_precomp=None, means2D=None, culling=None, lbs=None, warped=None):
    """Allocate outputs and launch ``fsgs_preprocess_forward``.  Returns the dict of outputs (no sync)."""
    P = opacities.shape[0]
    gx, gy = _tiles(W, H)
    has_rest = sh_rest is not None and sh_rest.numel() > 0
    o = _alloc_preprocess_outputs(P, gx * gy, opacities.device, sh_degree, shs, means2D, trans_precomp)
    a = _lib.PreprocessArgs()
    a.P, a.W, a.H, a.sh_degree = P, W, H, sh_degree
    a.n_dc = shs.shape[1] if sh_degree >= 0 else 1
    a.n_rest = sh_rest.shape[1] if has_rest else 0
    a.means, a.scales, a.rots = _ptr(means3D), _ptr(scales), _ptr(rotations)
    a.opac, a.shs, a.sh_rest = _ptr(opacities), _ptr(shs), _ptr(sh_rest if has_rest else None)
    a.Tw2v, a.Tv2s, a.campos = _ptr(Tw2v), _ptr(Tv2s), _ptr(campos)
    a.trans_precomp, a.culling = _ptr(trans_precomp), _ptr(culling)
    if lbs is not None:
        a.lbs = ctypes.pointer(lbs)
        a.warped_means, a.warped_scales, a.warped_rots = (_ptr(t) for t in warped)
    a.means2D, a.colors, a.trans_mat = _ptr(o["means2D"]), _ptr(o["colors"]), _ptr(o["trans_mat"])
    a.inverse_m, a.normal_opacity, a.depths = _ptr(o["inverse_m"]), _ptr(o["normal_opacity"]), _ptr(o["depths"])
    a.radii, a.tiles_touched, a.records = _ptr(o["radii"]), _ptr(o["tiles_touched"]), _ptr(o["records"])
    a.tile_counts, a.counters = _ptr(o["tile_counts"]), _ptr(o["counters"])
    check(lib().fsgs_preprocess_forward(ctypes.byref(a), _stream()), "fsgs_preprocess_forward")
    return o


def bin_launch(W, H, o, opacities, capacity):
    """Launch ``fsgs_bin_tiles`` into freshly allocated ``ranges`` / ``point_list[capacity]`` / ``tile_order``."""
    dev = opacities.device
    gx, gy = _tiles(W, H)
    T = gx * gy
    ranges = torch.empty(T, 2, device=dev, dtype=torch.int64)
    point_list = torch.empty(capacity, device=dev, dtype=torch.int32)
    tile_order = torch.empty(T, device=dev, dtype=torch.int32)
    ws_bytes = lib().fsgs_bin_workspace_bytes(W, H, capacity)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
    b = _lib.BinArgs()
    b.P, b.W, b.H = opacities.shape[0], W, H
    b.means2D, b.inverse_m, b.depths, b.opac = _ptr(o["means2D"]), _ptr(o["inverse_m"]), _ptr(o["depths"]), _ptr(opacities)
    b.radii, b.tile_counts, b.counters = _ptr(o["radii"]), _ptr(o["tile_counts"]), _ptr(o["counters"])
    b.capacity, b.point_list, b.ranges, b.tile_order = capacity, _ptr(point_list), _ptr(ranges), _ptr(tile_order)
    b.workspace, b.workspace_bytes = _ptr(ws), ws_bytes
    check(lib().fsgs_bin_tiles(ctypes.byref(b), _stream()), "fsgs_bin_tiles")
    return ranges, point_list, tile_order


def gs_2d_fast_preprocess_forward(W, H, sh_degree, is_opengl, means3D, scales, rotations, opacities, shs, sh_rest,
                                  Tw2v, Tv2c, Tv2s, cam_pos, trans_precomp, means2D, culling, debug=False):
    """``GS_2D_fast_preprocess_forward`` (src/gaussian_splatting/gs_2d_fast_preprocess.cu:611-782).

    Returns ``[means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list]``;
    ``point_list`` has one slot per tile of every splat's rectangle: real pairs first, sorted per tile by
    (depth bits, Gaussian index), then -1 padding.  ``is_opengl`` and ``Tv2c`` are accepted and, as in the
    reference, not read.  One 16-byte device-to-host read sizes ``point_list``; ``debug`` adds nothing.
    """
    W, H, sh_degree = int(W), int(H), int(sh_degree)
    _check_input(means3D, "means3D")
    _need(means3D.dim() == 2 and means3D.shape[-1] == 3, "Error shape for means3D")
    P = means3D.shape[0]
    _check_input(scales, "scales", (P, 2))
    _check_input(rotations, "rotations", (P, 4))
    _check_input(opacities, "opacities", (P, 1))
    _check_input(shs, "shs")
    has_rest = sh_rest is not None and sh_rest.numel() > 0
    nb = (1 + sh_degree) ** 2
    if has_rest:
        _check_input(sh_rest, "sh_rest")
        _need(sh_rest.dim() == 3 and sh_rest.shape[0] == P and sh_rest.shape[1] >= nb - 1 and sh_rest.shape[2] == 3,
              "Error shape for sh features")
    elif sh_degree >= 0:
        _need(shs.dim() == 3 and shs.shape[0] == P and shs.shape[1] >= nb and shs.shape[2] == 3,
              "Error shape for sh features")
    if sh_degree < 0:
        _need(tuple(shs.shape) == (P, 3), "shs have error shape")
    _check_input(Tw2v, "Tw2v", (4, 4))
    _check_input(Tv2c, "Tv2c", (4, 4))
    _check_input(Tv2s, "Tv2s", (3, 3))
    _check_input(cam_pos, "cam_pos", (3,))
    if means2D is not None:
        _check_input(means2D, "means2D", (P, 2))
    if culling is not None:
        _check_input(culling, "culling", (P,), torch.bool)
    if trans_precomp is not None:
        _check_input(trans_precomp, "trans_precomp", (P, 3, 3))
    _need(sh_degree <= 7, "SH degree above 7 is not supported (neither by the reference)")
    o = preprocess_launch(W, H, sh_degree, means3D, scales, rotations, opacities, shs, sh_rest, Tw2v, Tv2s, cam_pos,
                          trans_precomp, means2D, culling)
    n_slots = int(o["counters"][0].item()) if P > 0 else 0  # the reference blocks here too (:729)
    ranges, point_list, tile_order = bin_launch(W, H, o, opacities, n_slots)
    keep = (o["means2D"], o["colors"], o["trans_mat"], o["inverse_m"], o["normal_opacity"])
    point_list._fsgs_aux = RenderAux(o["records"], tile_order, keep)
    return [o["means2D"], o["colors"], o["trans_mat"], o["inverse_m"], o["normal_opacity"], o["depths"], o["radii"],
            ranges, point_list]


def _records_for(means2D, colors, normal_opacity, trans_mat, inverse_m, point_list):
    """Packed records + tile order: taken from ``point_list`` when it carries them for these very tensors."""
    keep = (means2D, colors, trans_mat, inverse_m, normal_opacity)
    aux = getattr(point_list, "_fsgs_aux", None)
    if aux is not None and aux.records is not None and aux.matches(keep):
        return aux.records, aux.tile_order
    P = colors.shape[0]
    records = torch.empty(P, REC, device=colors.device, dtype=torch.float32)
    check(lib().fsgs_pack_records(P, _ptr(means2D), _ptr(colors), _ptr(normal_opacity), _ptr(trans_mat),
                                  _ptr(inverse_m), _ptr(records), _stream()), "fsgs_pack_records")
    return records, None


def render_forward_launch(W, H, near_n, far_n, only_image, P, records, point_list, ranges, tile_order,
                          trans_mat_t2=None, accum_max_count=None, accum_weights_p=None, accum_weights_count=None,
                          counters=None):
    dev = ranges.device
    f32 = dict(device=dev, dtype=torch.float32)
    pixel_colors = torch.empty(3, H, W, **f32)
    pixel_opacity = torch.empty(H, W, **f32)
    n_contrib = torch.empty(2, H, W, device=dev, dtype=torch.int32)
    pixel_extras = None if only_image else torch.empty(8, H, W, **f32)
    pixel_flow = torch.empty(H, W, 2, **f32) if (not only_image and trans_mat_t2 is not None) else None
    a = _lib.RenderArgs()
    a.P, a.W, a.H, a.near_n, a.far_n, a.only_image = P, W, H, near_n, far_n, int(bool(only_image))
    a.records, a.point_list, a.ranges, a.tile_order = _ptr(records), _ptr(point_list), _ptr(ranges), _ptr(tile_order)
    a.trans_mat_t2 = _ptr(trans_mat_t2 if not only_image else None)
    a.out_color, a.out_opacity, a.out_extras = _ptr(pixel_colors), _ptr(pixel_opacity), _ptr(pixel_extras)
    a.out_flow, a.n_contrib = _ptr(pixel_flow), _ptr(n_contrib)
    a.accum_max_count, a.accum_weights_p = _ptr(accum_max_count), _ptr(accum_weights_p)
    a.accum_weights_count = _ptr(accum_weights_count)
    a.counters = _ptr(counters)  # a truncated list (overflow counter set) poisons the frame with NaN
    check(lib().fsgs_render_forward(ctypes.byref(a), _stream()), "fsgs_render_forward")
    return pixel_colors, pixel_opacity, pixel_extras, pixel_flow, n_contrib


def GS_2D_fast_render_forward(width, height, near_n, far_n, only_image, means2D, colors, normal_opacity, trans_mat,
                              inverse_m, point_list, ranges, trans_mat_t2=None, accum_max_count=None,
                              accum_weights_p=None, accum_weights_count=None, per_tile_bucket_offset=None):
    """``GS_2D_fast_render_forward`` (src/gaussian_splatting/gs_2d_fast_redner.cu:839-953).

    Returns ``[pixel_colors[3,H,W], pixel_opacity[H,W], pixel_extras[8,H,W]|None, pixel_flow[H,W,2]|None,
    n_contrib[2,H,W]]``.  With ``per_tile_bucket_offset`` (the reference's bucketed backward, which this library
    does not need) five placeholders are appended so that callers unpacking ten values keep working.
    """
    W, H = int(width), int(height)
    _check_input(colors, "colors")
    _need(colors.dim() == 2, "The ndim of colors must be 2")
    P = colors.shape[0]
    _check_input(trans_mat, "trans_mat", (P, 3, 3))
    _check_input(inverse_m, "inverse_m", (P, 3, 3))
    _check_input(ranges, "ranges", dtype=torch.int64)
    _check_input(point_list, "point_list", dtype=torch.int32)
    dev = colors.device
    if accum_max_count is not None:
        _check_input(accum_max_count, "accum_max_count", (P,), torch.int32)
    if accum_weights_p is not None:
        _check_input(accum_weights_p, "accum_weights_p", (P,))
    if accum_weights_count is not None:
        _check_input(accum_weights_count, "accum_weights_count", (P,), torch.int32)
    if trans_mat_t2 is not None:
        _check_input(trans_mat_t2, "trans_mat_t2", (P, 3, 3))
    means2D, normal_opacity = means2D.contiguous(), normal_opacity.contiguous()
    if P == 0:
        z = dict(device=dev, dtype=torch.float32)
        outs = [torch.zeros(3, H, W, **z), torch.zeros(H, W, **z), None if only_image else torch.zeros(8, H, W, **z),
                None, torch.zeros(2, H, W, device=dev, dtype=torch.int32)]
    else:
        records, tile_order = _records_for(means2D, colors, normal_opacity, trans_mat, inverse_m, point_list)
        outs = list(render_forward_launch(W, H, float(near_n), float(far_n), bool(only_image), P, records, point_list,
                                          ranges, tile_order, trans_mat_t2, accum_max_count, accum_weights_p,
                                          accum_weights_count))
    if per_tile_bucket_offset is not None:
        gx, gy = _tiles(W, H)
        empty = torch.empty(0, device=dev, dtype=torch.float32)
        outs += [torch.zeros(gy, gx, device=dev, dtype=torch.int32), torch.empty(0, device=dev, dtype=torch.int32),
                 empty, empty, empty]
    return outs


def render_backward_launch(W, H, near_n, far_n, P, records, point_list, ranges, tile_order, trans_mat_t2,
                           out_opacity, out_extras, n_contrib, dL_dcolor, dL_dopacity, dL_dextras, dL_dflow):
    dev = ranges.device
    # one allocation, five views: colours 3, mean2D 2, trans_mat 9, inverse_m 9, normal+opacity 4.  Every view starts
    # on a 256-byte boundary whatever P is: the preprocess adjoint reads them with float2 / float4 loads
    Pp = (P + 63) & ~63
    buf = torch.empty(Pp * 27, device=dev, dtype=torch.float32)
    g_col = buf[:3 * P].view(P, 3)
    g_m2d = buf[3 * Pp:3 * Pp + 2 * P].view(P, 2)
    g_tm = buf[5 * Pp:5 * Pp + 9 * P].view(P, 3, 3)
    g_im = buf[14 * Pp:14 * Pp + 9 * P].view(P, 3, 3)
    g_no = buf[23 * Pp:23 * Pp + 4 * P].view(P, 4)
    a = _lib.RenderBwdArgs()
    a.P, a.W, a.H, a.near_n, a.far_n = P, W, H, near_n, far_n
    a.records, a.point_list, a.ranges, a.tile_order = _ptr(records), _ptr(point_list), _ptr(ranges), _ptr(tile_order)
    a.trans_mat_t2 = _ptr(trans_mat_t2)
    a.out_opacity, a.out_extras, a.n_contrib = _ptr(out_opacity), _ptr(out_extras), _ptr(n_contrib)
    a.dL_dcolor, a.dL_dopacity, a.dL_dextras, a.dL_dflow = _ptr(dL_dcolor), _ptr(dL_dopacity), _ptr(dL_dextras), _ptr(dL_dflow)
    a.dL_dcolors, a.dL_dmeans2D, a.dL_dtrans_mat = _ptr(g_col), _ptr(g_m2d), _ptr(g_tm)
    a.dL_dinverse_m, a.dL_dnormal_opacity = _ptr(g_im), _ptr(g_no)
    check(lib().fsgs_render_backward(ctypes.byref(a), _stream()), "fsgs_render_backward")
    return g_col, g_m2d, g_tm, g_im, g_no


def GS_2D_fast_render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, trans_mat2, images,
                               out_opacity, out_others, out_flows, dL_dout_color, dL_dout_opacity, dL_dothers,
                               dL_dout_flow, ranges, point_list, n_contrib, near_n, far_n,
                               per_tile_bucket_offset=None, bucket_to_tile=None, max_contrib=None, sampled_T=None,
                               sampled_acc=None, sampled_aux=None):
    """``GS_2D_fast_render_backward`` (src/gaussian_splatting/gs_2d_fast_redner.cu:955-1074).

    Returns ``[dL_dcolors, dL_dmeans2D, dL_dtrans_mat, dL_dinverse_m, dL_dnormal_opacity]`` with the semantics of
    the reference's per-pixel kernel (the one training reaches); the six bucket arguments are accepted and unused.
    Upstream gradients may be non-contiguous (the reference calls ``.contiguous()`` on them too).
    """
    _need(dL_dout_color.is_cuda and dL_dout_opacity.is_cuda, "gradients must be CUDA tensors")
    P = means2D.shape[0]
    H, W = dL_dout_color.shape[1], dL_dout_color.shape[2]
    dev = out_opacity.device
    if P == 0:
        z = dict(device=dev, dtype=torch.float32)
        return [torch.zeros(0, 3, **z), torch.zeros(0, 2, **z), torch.zeros(0, 3, 3, **z), torch.zeros(0, 3, 3, **z),
                torch.zeros(0, 4, **z)]
    means2D, normal_opacity, colors = means2D.contiguous(), normal_opacity.contiguous(), colors.contiguous()
    records, tile_order = _records_for(means2D, colors, normal_opacity, trans_mat, inverse_m, point_list)
    aux = out_others is not None and dL_dothers is not None
    flow = aux and dL_dout_flow is not None and trans_mat2 is not None
    g = render_backward_launch(
        W, H, float(near_n), float(far_n), P, records, point_list.contiguous(), ranges.contiguous(), tile_order,
        trans_mat2 if flow else None, out_opacity.contiguous(), out_others.contiguous() if aux else None,
        n_contrib.contiguous(), dL_dout_color.contiguous(),
        # the reference's kernel without auxiliary channels ignores the opacity gradient (gs_2d_fast_redner.cu:338-341)
        dL_dout_opacity.contiguous() if aux else None,
        dL_dothers.contiguous() if aux else None, dL_dout_flow.contiguous() if flow else None)
    return list(g)


def gs_2d_fast_preprocess_backward(W, H, sh_degree, is_opengl, means3D, scales, rotations, opacities, shs, sh_rest,
                                   Tw2v, Tv2s, cam_pos, trans_mat, radii, colors, normal_opacity, grad_mean2D,
                                   grad_trans, grad_inv_m, grad_depth, grad_colors, grad_normals, grad_means3D,
                                   grad_scales, grad_rotations, grad_opacities, grad_shs, grad_sh_rest,
                                   grad_Tw2v=None, grad_campos=None):
    """``GS_2D_fast_preprocess_backward`` (src/gaussian_splatting/gs_2d_fast_preprocess.cu:784-859): fills the
    caller's ``grad_*`` tensors in place, overwrites ``grad_mean2D`` with the densification proxy, returns None.
    Camera gradients are not produced (the reference leaves them untouched as well)."""
    W, H, sh_degree = int(W), int(H), int(sh_degree)
    P = means3D.shape[0]
    for t, n in ((grad_mean2D, "grad_mean2D"), (grad_normals, "grad_normals"), (grad_means3D, "grad_means3D"),
                 (grad_trans, "grad_trans"), (grad_opacities, "grad_opacities")):
        _check_input(t, n)
    _check_input(grad_means3D, "grad_means3D", (P, 3))
    _check_input(grad_opacities, "grad_opacities", (P, 1))
    _need(grad_scales is not None and grad_rotations is not None, "grad_scales / grad_rotations are required")
    _check_input(grad_scales, "grad_scales", (P, 2))
    _check_input(grad_rotations, "grad_rotations", (P, 4))
    if grad_colors is not None:
        _check_input(grad_colors, "grad_colors")
    if grad_shs is not None:
        _need(colors is not None, "shs and clamped must not be None when need grad_shs")
        _check_input(grad_shs, "grad_shs")
    if grad_sh_rest is not None:
        _check_input(grad_sh_rest, "grad_sh_rest")
    _need(trans_mat is not None, "trans_mat is required")
    has_rest = sh_rest is not None and sh_rest.numel() > 0
    a = _lib.PreprocessBwdArgs()
    a.P, a.W, a.H, a.sh_degree = P, W, H, sh_degree
    a.n_dc = shs.shape[1] if sh_degree >= 0 else 1
    a.n_rest = sh_rest.shape[1] if has_rest else 0
    a.means, a.scales, a.rots = _ptr(means3D), _ptr(scales), _ptr(rotations)
    a.shs, a.sh_rest = _ptr(shs), _ptr(sh_rest if has_rest else None)
    a.Tw2v, a.Tv2s, a.campos = _ptr(Tw2v), _ptr(Tv2s), _ptr(cam_pos)
    a.trans_mat, a.colors, a.radii = _ptr(trans_mat), _ptr(colors), _ptr(radii)
    a.grad_means2D, a.grad_trans_mat, a.grad_inverse_m = _ptr(grad_mean2D), _ptr(grad_trans), _ptr(grad_inv_m)
    a.grad_colors, a.grad_normal_opacity = _ptr(grad_colors), _ptr(grad_normals)
    a.grad_means, a.grad_scales, a.grad_rots = _ptr(grad_means3D), _ptr(grad_scales), _ptr(grad_rotations)
    a.grad_opac, a.grad_shs, a.grad_sh_rest = _ptr(grad_opacities), _ptr(grad_shs), _ptr(grad_sh_rest)
    check(lib().fsgs_preprocess_backward(ctypes.byref(a), _stream()), "fsgs_preprocess_backward")
    return None


def gs_2d_fast_compute_transmat_forward(means3D, scales, rotations, Tw2v, Tv2s):
    """``gs_2d_fast_compute_trans_mat_forward`` (gs_2d_fast_preprocess.cu:871-909) -> ``(trans_mat, normals)``, float32
    or float64 like the reference (``AT_DISPATCH_FLOATING_TYPES``, :889); the camera matrices are taken in the
    inputs' type.  They stay on the device (the reference copies them to the host, which synchronises)."""
    P = means3D.shape[0]
    dt = means3D.dtype
    _need(dt in (torch.float32, torch.float64), "means3D must be a float32 or float64 tensor")
    _check_input(means3D, "means3D", (P, 3), dt)
    _check_input(scales, "scales", (P, 2), dt)
    _check_input(rotations, "rotations", (P, 4), dt)
    Tw2v, Tv2s = Tw2v.to(dt).contiguous(), Tv2s.to(dt).contiguous()
    _check_input(Tw2v, "Tw2v", (4, 4), dt)
    _check_input(Tv2s, "Tv2s", (3, 3), dt)
    trans_mat = torch.empty(P, 3, 3, device=means3D.device, dtype=dt)
    normals = torch.empty(P, 3, device=means3D.device, dtype=dt)
    fn = lib().fsgs_transmat_forward if dt == torch.float32 else lib().fsgs_transmat_forward_f64
    check(fn(P, _ptr(means3D), _ptr(scales), _ptr(rotations), _ptr(Tw2v), _ptr(Tv2s), _ptr(trans_mat), _ptr(normals),
             _stream()), "fsgs_transmat_forward")
    return trans_mat, normals


def gs_2d_fast_compute_trans_mat_backward(means3D, scales, rotations, Tw2v, Tv2s, grad_matrix, grad_normals):
    """``gs_2d_fast_compute_trans_mat_backward`` (gs_2d_fast_preprocess.cu:923-958) ->
    ``[grad_means3D, grad_scales, grad_rotations]``, float32 or float64 (:936)."""
    P = means3D.shape[0]
    dt = means3D.dtype
    _need(dt in (torch.float32, torch.float64), "means3D must be a float32 or float64 tensor")
    _check_input(grad_matrix, "grad_matrix", (P, 3, 3), dt)
    _check_input(grad_normals, "grad_normals", (P, 3), dt)
    kw = dict(device=means3D.device, dtype=dt)
    g_m, g_s, g_r = torch.empty(P, 3, **kw), torch.empty(P, 2, **kw), torch.empty(P, 4, **kw)
    fn = lib().fsgs_transmat_backward if dt == torch.float32 else lib().fsgs_transmat_backward_f64
    check(fn(P, _ptr(scales.to(dt).contiguous()), _ptr(rotations.to(dt).contiguous()), _ptr(Tw2v.to(dt).contiguous()),
             _ptr(Tv2s.to(dt).contiguous()), _ptr(grad_matrix), _ptr(grad_normals), _ptr(g_m), _ptr(g_s), _ptr(g_r),
             _stream()), "fsgs_transmat_backward")
    return [g_m, g_s, g_r]


def _batch_dims(x1, x2):
    _need(x1.is_cuda and x2.is_cuda, "cdist_top: this library has no CPU path; pass CUDA tensors")
    _need(x1.device == x2.device, "x1 and x2 must be same device")
    _need(x1.dtype in (torch.float32, torch.float64) and x2.dtype == x1.dtype,
          "cdist_top: float32 or float64, the same for both inputs")
    N, D, M = x1.shape[-2], x1.shape[-1], x2.shape[-2]
    _need(x2.shape[-1] == D, f"The dimenstion of point must be {D}")
    B = 1
    for n in x1.shape[:-2]:
        B *= n
    _need(x2.numel() == B * M * D, "The shape[:-2] of x2 must be same with x1")
    return B, N, M, D


def cdist_top(x1, x2, largest=False):
    """``cdist_top`` (src/other/cdist_top.cu:34-84) -> ``[distance[...,N], index[...,N] int64]``: for every row of
    ``x1`` the nearest (or farthest) row of ``x2``, Euclidean distance.  Exact ties: nearest -> last index."""
    B, N, M, D = _batch_dims(x1, x2)
    x1, x2 = x1.contiguous(), x2.contiguous()
    dist = torch.empty(x1.shape[:-1], device=x1.device, dtype=x1.dtype)
    index = torch.empty(x1.shape[:-1], device=x1.device, dtype=torch.int64)
    if dist.numel() == 0:
        return [dist, index]
    fn = lib().fsgs_cdist_top_f64 if x1.dtype == torch.float64 else lib().fsgs_cdist_top
    check(fn(B, N, M, D, _ptr(x1), _ptr(x2), int(bool(largest)), _ptr(dist), _ptr(index), _stream()), "fsgs_cdist_top")
    return [dist, index]


def cdist_top_backward(x1, x2, distance, index, grad_dist):
    """``cdist_top_backward`` (src/other/cdist_top.cu:107-154) -> ``[grad_x1, grad_x2]``."""
    B, N, M, D = _batch_dims(x1, x2)
    x1, x2 = x1.contiguous(), x2.contiguous()
    g1, g2 = torch.empty_like(x1), torch.empty_like(x2)
    fn = lib().fsgs_cdist_top_backward_f64 if x1.dtype == torch.float64 else lib().fsgs_cdist_top_backward
    check(fn(B, N, M, D, _ptr(x1), _ptr(x2), _ptr(distance.to(x1.dtype).contiguous()), _ptr(index.contiguous()),
             _ptr(grad_dist.to(x1.dtype).contiguous()), _ptr(g1), _ptr(g2), _stream()), "fsgs_cdist_top_backward")
    return [g1, g2]


def AdamMasksedUpdated(param, param_grad, exp_avg, exp_avg_sq, tiles_touched, lr, b1, b2, eps, N, M):
    """``AdamMasksedUpdated`` (src/other/adam_masked_update.cu:30-36): in-place Adam step on the rows of a
    ``[N, M]`` parameter whose ``tiles_touched`` (bool [N]) entry is set."""
    for t, n in ((param, "param"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        _need(t.is_cuda and t.is_contiguous() and t.dtype == torch.float32, f"{n} must be a contiguous CUDA float tensor")
    _need(tiles_touched.dtype in (torch.bool, torch.uint8), "tiles_touched must be bool")
    check(lib().fsgs_adam_masked(_ptr(param), _ptr(param_grad.contiguous()), _ptr(exp_avg), _ptr(exp_avg_sq),
                                 _ptr(tiles_touched.contiguous()), float(lr), float(b1), float(b2), float(eps), int(N),
                                 int(M), _stream()), "fsgs_adam_masked")
    return None


def knn(x, c, K, method="auto"):
    """Exact K nearest rows of ``c`` [M,3] for each row of ``x`` [N,3]: ``(squared distance [N,K], index [N,K] int64)``
    ascending by (distance, index).  ``method``: ``"brute"`` evaluates every pair, ``"grid"`` searches a uniform grid
    over ``c`` (same results bit for bit, far fewer evaluations), ``"auto"`` takes the grid from 1024 control points
    up (measured: 0.08 against 0.05 ms at 512 control points, 1.8 against 6.3 ms at 4096)."""
    _need(x.is_cuda and c.is_cuda and x.dtype == torch.float32 and c.dtype == torch.float32, "knn: CUDA float32 only")
    _need(x.dim() == 2 and c.dim() == 2 and x.shape[1] == 3 and c.shape[1] == 3, "knn: [N,3] and [M,3] expected")
    x, c = x.contiguous(), c.contiguous()
    N, M = x.shape[0], c.shape[0]
    d2 = torch.empty(N, K, device=x.device, dtype=torch.float32)
    idx = torch.empty(N, K, device=x.device, dtype=torch.int64)
    _need(method in ("auto", "brute", "grid"), "knn: method is auto, brute or grid")
    if method == "grid" or (method == "auto" and M >= 1024):
        n = int(lib().fsgs_knn_grid_workspace_bytes(M))
        ws = torch.empty(n, dtype=torch.uint8, device=x.device)
        check(lib().fsgs_knn_grid(N, M, int(K), _ptr(x), _ptr(c), _ptr(d2), _ptr(idx), _ptr(ws), n, _stream()),
              "fsgs_knn_grid")
    else:
        check(lib().fsgs_knn(N, M, int(K), _ptr(x), _ptr(c), _ptr(d2), _ptr(idx), _stream()), "fsgs_knn")
    return d2, idx


def compact_rows(tensors, keep):
    """Keep the rows (dim 0) of every tensor in ``tensors`` whose entry in ``keep`` (bool [N]) is set, in order:
    the result of ``[t[keep] for t in tensors]`` with one plan, one host read of the row count and one gather launch
    per 24 tensors (the reference indexes each parameter and Adam moment separately,
    fast_2d_gs/gaussian_splatting.py:495-548)."""
    N = keep.shape[0]
    _need(keep.is_cuda and keep.dtype in (torch.bool, torch.uint8) and keep.dim() == 1, "keep must be a CUDA bool [N]")
    for t in tensors:
        _need(t.is_cuda and t.shape[0] == N and t.element_size() in (4, 8), "rows of 4- or 8-byte elements, N each")
    keep8 = keep.contiguous().view(torch.uint8)
    ws = torch.empty(int(lib().fsgs_compact_workspace_bytes(N)), dtype=torch.uint8, device=keep.device)
    count = torch.empty(1, dtype=torch.int64, device=keep.device)
    check(lib().fsgs_compact_plan(N, _ptr(keep8), _ptr(ws), ws.numel(), _ptr(count), _stream()), "fsgs_compact_plan")
    n = int(count)  # the one synchronisation: the outputs are sized by it
    src = [t.contiguous() for t in tensors]
    out = [torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for t in src]
    for i in range(0, len(src), 24):
        chunk = list(zip(src[i:i + 24], out[i:i + 24]))
        arr = (_lib.RowTensor * len(chunk))()
        for k, (a, b) in enumerate(chunk):
            arr[k].src, arr[k].dst = a.data_ptr(), b.data_ptr()
            arr[k].row_words = (a.numel() // max(N, 1)) * (a.element_size() // 4)
        if n > 0 and N > 0:
            check(lib().fsgs_compact_rows(len(chunk), arr, N, _ptr(keep8), _ptr(ws), _stream()), "fsgs_compact_rows")
    return out


def gather_rows(tensors, index):
    """``[t[index] for t in tensors]`` in one launch per 24 tensors, with ``index`` int32 [n_out] and negative entries
    giving zero rows (fresh optimiser state for new Gaussians)."""
    _need(index.is_cuda and index.dtype == torch.int32 and index.dim() == 1, "index must be a CUDA int32 vector")
    n = index.shape[0]
    src = [t.contiguous() for t in tensors]
    for t in src:
        _need(t.is_cuda and t.element_size() in (4, 8) and t.shape[0] > 0, "rows of 4- or 8-byte elements")
    out = [torch.empty((n,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device) for t in src]
    for i in range(0, len(src), 24):
        chunk = list(zip(src[i:i + 24], out[i:i + 24]))
        arr = (_lib.RowTensor * len(chunk))()
        for k, (a, b) in enumerate(chunk):
            arr[k].src, arr[k].dst = a.data_ptr(), b.data_ptr()
            arr[k].row_words = (a.numel() // a.shape[0]) * (a.element_size() // 4)
        if n > 0:
            check(lib().fsgs_gather_rows(len(chunk), arr, n, _ptr(index), _stream()), "fsgs_gather_rows")
    return out


SH_SOURCE_FLOATS = 7  # a row of the SH-gradient factors: colour gradient 3 | view direction 3 | visibility 1


def sh_grad_from_views(sh_source, order, sh_degree, g_sh_dc, g_sh_rest, visible=None):
    """Summed SH gradient of several views from their factors.  ``sh_source [S,P,7]``: per slot and Gaussian the clamped
    colour gradient, the unit view direction and the view's visibility (1 / 0, -inf from an overflowed view), as the
    training engine's backward writes them (``sh_source=``); slots of zeros add nothing.  ``order``: the slots in
    summation order.  Writes ``g_sh_dc [P,1,3]``, ``g_sh_rest [P,n_rest,3]`` and, when given, ``visible [P]`` = the sum
    of the slots' visibility entries (reference SH adjoint: utils/ops_3d/spherical_harmonics.py:242-302)."""
    _need(sh_source.is_cuda and sh_source.is_contiguous() and sh_source.dtype == torch.float32 and sh_source.dim() == 3
          and sh_source.shape[2] == SH_SOURCE_FLOATS, "sh_source: contiguous float32 CUDA [S,P,7]")
    S, P = int(sh_source.shape[0]), int(sh_source.shape[1])
    _need(len(order) <= S, "more slots in order than in sh_source")
    for t in (g_sh_dc, g_sh_rest, visible):
        _need(t is None or (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32), "outputs: float32 CUDA")
    n_rest = 0 if g_sh_rest is None else int(g_sh_rest.shape[1])
    arr = (ctypes.c_int32 * max(len(order), 1))(*[int(o) for o in order])
    check(lib().fsgs_sh_grad_from_views(P, int(sh_degree), n_rest, len(order), arr, _ptr(sh_source),
                                        P * SH_SOURCE_FLOATS, _ptr(g_sh_dc), _ptr(g_sh_rest), _ptr(visible), _stream()),
          "fsgs_sh_grad_from_views")


def densify_select(accum, denom, scaling_raw, grad_threshold, scale_threshold):
    """uint8 flags [P]: 1 clone, 2 split, 0 neither (gaussian_splatting.py:581-588, 608-613)."""
    P = scaling_raw.shape[0]
    flags = torch.empty(P, dtype=torch.uint8, device=scaling_raw.device)
    check(lib().fsgs_densify_select(P, _ptr(accum.contiguous()), _ptr(denom.contiguous()), _ptr(scaling_raw.contiguous()),
                                    float(grad_threshold), float(scale_threshold), _ptr(flags), _stream()),
          "fsgs_densify_select")
    return flags


def split_children(parent, z, xyz, scaling_raw, rotation_raw, N, xyz_out, scaling_out):
    """Positions and log-scales of the split children into ``xyz_out [n,3]`` / ``scaling_out [n,2]`` (contiguous views
    are fine); ``parent`` int32 [n], ``z`` [n,2] standard-normal draws."""
    n = parent.shape[0]
    _need(xyz_out.is_contiguous() and scaling_out.is_contiguous() and z.is_contiguous(), "contiguous outputs and noise")
    check(lib().fsgs_split_children(n, int(N), _ptr(parent), _ptr(z), _ptr(xyz.contiguous()),
                                    _ptr(scaling_raw.contiguous()), _ptr(rotation_raw.contiguous()), _ptr(xyz_out),
                                    _ptr(scaling_out), _stream()), "fsgs_split_children")


def densify_stats(viewspace_grad, radii, accum, denom, max_radii):
    check(lib().fsgs_densify_stats(radii.shape[0], _ptr(viewspace_grad), _ptr(radii), _ptr(accum), _ptr(denom),
                                   _ptr(max_radii), _stream()), "fsgs_densify_stats")


def _ssim_check(img1, img2):
    _need(img1.dim() == 4 and img1.shape == img2.shape, "fusedssim: images must be [B,C,H,W] of equal shape")
    for t, n in ((img1, "img1"), (img2, "img2")):
        _need(t.is_cuda and t.dtype == torch.float32, f"{n} must be a float32 CUDA tensor")


def fusedssim(C1, C2, img1, img2, train=True):
    """``fusedssim`` (src/other/structural_similarity.cu:340-361) -> ``(ssim_map, dm_dmu1, dm_dsigma1_sq,
    dm_dsigma12)``; the three derivative maps are empty tensors when ``train`` is false."""
    _ssim_check(img1, img2)
    img1, img2 = img1.contiguous(), img2.contiguous()
    B, C, H, W = img1.shape
    ssim_map = torch.empty_like(img1)
    d = [torch.empty_like(img1) for _ in range(3)] if train else [None] * 3
    check(lib().fsgs_ssim_forward(B, C, H, W, float(C1), float(C2), _ptr(img1), _ptr(img2), _ptr(ssim_map),
                                  _ptr(d[0]), _ptr(d[1]), _ptr(d[2]), None, _stream()), "fsgs_ssim_forward")
    if not train:
        d = [torch.empty(0) for _ in range(3)]
    return ssim_map, d[0], d[1], d[2]


def fusedssim_backward(C1, C2, img1, img2, dL_dmap, dm_dmu1, dm_dsigma1_sq, dm_dsigma12):
    """``fusedssim_backward`` (structural_similarity.cu:363-381) -> ``dL_dimg1``."""
    _ssim_check(img1, img2)
    img1, img2, dL_dmap = img1.contiguous(), img2.contiguous(), dL_dmap.contiguous()
    _need(dL_dmap.shape == img1.shape and dm_dmu1.shape == img1.shape, "fusedssim_backward: shape mismatch")
    B, C, H, W = img1.shape
    out = torch.empty_like(img1)
    check(lib().fsgs_ssim_backward(B, C, H, W, float(C1), float(C2), _ptr(img1), _ptr(img2), _ptr(dL_dmap), 0.0,
                                   0.0, _ptr(dm_dmu1.contiguous()), _ptr(dm_dsigma1_sq.contiguous()),
                                   _ptr(dm_dsigma12.contiguous()), _ptr(out), _stream()), "fsgs_ssim_backward")
    return out


# the names the reference looks up with get_C_function(...) (fast_2d_gs/_C/__init__.py:41-42): the nine operators
# of the rendering path and the two of the SSIM loss
REFERENCE_OPS = {f.__name__: _Op(f) for f in (
    gs_2d_fast_preprocess_forward, gs_2d_fast_preprocess_backward, GS_2D_fast_render_forward,
    GS_2D_fast_render_backward, gs_2d_fast_compute_transmat_forward, gs_2d_fast_compute_trans_mat_backward,
    cdist_top, cdist_top_backward, AdamMasksedUpdated, fusedssim, fusedssim_backward)}
