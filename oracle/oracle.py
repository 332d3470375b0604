"""ctypes face of ``libfsgs_oracle.so`` -- the CPU restatement of the reference hot path.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke test and by the CPU-baseline leg of
``bench.py``; the product never imports it.

Functions take/return CPU ``torch`` tensors and mirror the positional order of the reference operators
(``fast_2d_gs/_C/src/gaussian_splatting/gs_2d_fast_preprocess.cu:611-618,781``,
``gs_2d_fast_redner.cu:839-843,955-968``, ``src/other/cdist_top.cu:156-159``,
``src/other/adam_masked_update.cu:30-31``).
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libfsgs_oracle.so")
        src = os.path.join(_HERE, "fsgs_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_bin.restype = ctypes.c_int64
        _LIB.orc_bin_size.restype = ctypes.c_int64
        _LIB.orc_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    """Threads for the oracle's parallel loops from now on (overrides an inherited OMP_NUM_THREADS)."""
    lib().orc_set_num_threads(ctypes.c_int(int(n)))


def _p(t):
    if t is None:
        return ctypes.c_void_p(0)
    assert t.device.type == "cpu" and t.is_contiguous(), "oracle wants contiguous CPU tensors"
    return ctypes.c_void_p(t.data_ptr())


def _f(t):
    return None if t is None else t.detach().to(torch.float32).contiguous()


_cf = ctypes.c_float
_ci = ctypes.c_int


def _sh_dims(sh_degree, shs, sh_rest):
    if sh_degree < 0:
        return 1, 0
    n_dc = shs.shape[1]
    n_rest = sh_rest.shape[1] if sh_rest is not None and sh_rest.numel() > 0 else 0
    return n_dc, n_rest


def transmat(means, scales, rots, Tw2v, Tv2s):
    P = means.shape[0]
    M = torch.zeros(P, 3, 3)
    n = torch.zeros(P, 3)
    lib().orc_transmat(_ci(P), _p(_f(means)), _p(_f(scales)), _p(_f(rots)), _p(_f(Tw2v)), _p(_f(Tv2s)), _p(M), _p(n))
    return M, n


def sh_basis(dirs, degree):
    """Real SH basis at unit directions [n,3] -> [n, (degree+1)^2], degree <= 7."""
    dirs = _f(dirs)
    n, nb = dirs.shape[0], (degree + 1) ** 2
    out = torch.zeros(n, nb)
    lib().orc_sh_basis(_ci(n), _ci(degree), _p(dirs), _p(out))
    return out


def preprocess_forward(W, H, sh_degree, means, scales, rots, opac, shs, sh_rest, Tw2v, Tv2s, campos, culling=None,
                       with_bin=True):
    """Returns the reference's nine outputs, then tiles_touched and the number of real (non padding) pairs."""
    P = means.shape[0]
    means, scales, rots, opac, shs = _f(means), _f(scales), _f(rots), _f(opac), _f(shs)
    sh_rest = _f(sh_rest) if sh_rest is not None and sh_rest.numel() > 0 else None
    n_dc, n_rest = _sh_dims(sh_degree, shs, sh_rest)
    means2D = torch.zeros(P, 2)
    colors = shs.clone() if sh_degree < 0 else torch.zeros(P, 3)
    trans_mat = torch.zeros(P, 3, 3)
    inverse_m = torch.zeros(P, 3, 3)
    normal_opacity = torch.zeros(P, 4)
    depths = torch.zeros(P)
    radii = torch.zeros(P, dtype=torch.int32)
    tiles = torch.zeros(P, dtype=torch.int32)
    cul = None if culling is None else culling.to(torch.uint8).contiguous()
    lib().orc_preprocess_fwd(_ci(P), _ci(W), _ci(H), _ci(sh_degree), _ci(n_dc), _ci(n_rest), _p(means), _p(scales),
                             _p(rots), _p(opac), _p(shs), _p(sh_rest), _p(_f(Tw2v)), _p(_f(Tv2s)), _p(_f(campos)),
                             _p(cul), _p(means2D), _p(colors), _p(trans_mat), _p(inverse_m), _p(normal_opacity),
                             _p(depths), _p(radii), _p(tiles))
    if not with_bin:
        return means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, None, None, tiles, 0
    ranges, point_list, n_real = bin_tiles(W, H, means2D, inverse_m, depths, opac, radii, tiles)
    return means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list, tiles, n_real


def bin_tiles(W, H, means2D, inverse_m, depths, opac, radii, tiles, want_keys=False):
    P = means2D.shape[0]
    T = ((W + 15) // 16) * ((H + 15) // 16)
    R = lib().orc_bin_size(_ci(P), _p(tiles))
    point_list = torch.zeros(R, dtype=torch.int32)
    ranges = torch.zeros(T, 2, dtype=torch.int64)
    keys = torch.zeros(R, dtype=torch.int64) if want_keys else None
    n_real = lib().orc_bin(_ci(P), _ci(W), _ci(H), _p(_f(means2D)), _p(_f(inverse_m)), _p(_f(depths)), _p(_f(opac)),
                           _p(radii), _p(tiles), _p(point_list), _p(ranges), _p(keys))
    if want_keys:
        return ranges, point_list, n_real, keys
    return ranges, point_list, n_real


def conic(inverse_m, opac, radii):
    P = inverse_m.shape[0]
    w6 = torch.zeros(P, 6)
    lib().orc_conic(_ci(P), _p(_f(inverse_m)), _p(_f(opac)), _p(radii.contiguous()), _p(w6))
    return w6


def render_forward(W, H, near, far, only_image, means2D, colors, normal_opacity, trans_mat, inverse_m, point_list,
                   ranges, trans_mat_t2=None, accum_max_count=None, accum_weights_p=None, accum_weights_count=None):
    aux = 0 if only_image else 1
    pc = torch.zeros(3, H, W)
    po = torch.zeros(H, W)
    pe = torch.zeros(8, H, W) if aux else None
    pf = torch.zeros(H, W, 2) if aux and trans_mat_t2 is not None else None
    nc = torch.zeros(2, H, W, dtype=torch.int32)
    lib().orc_blend_fwd(_ci(W), _ci(H), _cf(near), _cf(far), _ci(aux), _p(_f(means2D)), _p(_f(colors)),
                        _p(_f(normal_opacity)), _p(_f(trans_mat)), _p(_f(inverse_m)), _p(point_list.contiguous()),
                        _p(ranges.contiguous()), _p(_f(trans_mat_t2)), _p(pc), _p(po), _p(pe), _p(pf), _p(nc),
                        _p(accum_max_count), _p(accum_weights_p), _p(accum_weights_count))
    return pc, po, pe, pf, nc


def render_backward(means2D, normal_opacity, colors, trans_mat, inverse_m, trans_mat_t2, out_opacity, out_extras,
                    dL_dcolor, dL_dopacity, dL_dextras, dL_dflow, ranges, point_list, n_contrib, near, far):
    """Returns [dL_dcolors, dL_dmeans2D, dL_dtrans_mat, dL_dinverse_m, dL_dnormal_opacity] like the reference."""
    P = means2D.shape[0]
    H, W = out_opacity.shape
    g_m2d = torch.zeros(P, 2)
    g_col = torch.zeros(P, 3)
    g_no = torch.zeros(P, 4)
    g_tm = torch.zeros(P, 3, 3)
    g_im = torch.zeros(P, 3, 3)
    lib().orc_blend_bwd(_ci(W), _ci(H), _cf(near), _cf(far), _p(_f(means2D)), _p(_f(colors)), _p(_f(normal_opacity)),
                        _p(_f(trans_mat)), _p(_f(inverse_m)), _p(point_list.contiguous()), _p(ranges.contiguous()),
                        _p(_f(trans_mat_t2)), _p(_f(out_opacity)), _p(_f(out_extras)), _p(n_contrib.contiguous()),
                        _p(_f(dL_dcolor)), _p(_f(dL_dopacity)), _p(_f(dL_dextras)), _p(_f(dL_dflow)), _p(g_m2d),
                        _p(g_col), _p(g_no), _p(g_tm), _p(g_im))
    return g_col, g_m2d, g_tm, g_im, g_no


def preprocess_backward(W, H, sh_degree, means, scales, rots, shs, sh_rest, Tw2v, Tv2s, campos, trans_mat, radii,
                        colors, g_means2D, g_trans_mat, g_inverse_m, g_colors, g_normal_opacity, want_sh_grad=True):
    """Returns (g_means, g_scales, g_rots, g_opac, g_shs, g_sh_rest, g_means2D_proxy)."""
    P = means.shape[0]
    shs = _f(shs)
    sh_rest = _f(sh_rest) if sh_rest is not None and sh_rest.numel() > 0 else None
    n_dc, n_rest = _sh_dims(sh_degree, shs, sh_rest)
    g_means, g_scales, g_rots, g_opac = torch.zeros(P, 3), torch.zeros(P, 2), torch.zeros(P, 4), torch.zeros(P, 1)
    g_shs = torch.zeros_like(shs) if want_sh_grad and sh_degree >= 0 else None
    g_rest = torch.zeros_like(sh_rest) if want_sh_grad and sh_rest is not None and sh_degree >= 0 else None
    g_m2d = _f(g_means2D).clone()
    lib().orc_preprocess_bwd(_ci(P), _ci(W), _ci(H), _ci(sh_degree), _ci(n_dc), _ci(n_rest), _p(_f(means)),
                             _p(_f(scales)), _p(_f(rots)), _p(shs), _p(sh_rest), _p(_f(Tw2v)), _p(_f(Tv2s)),
                             _p(_f(campos)), _p(_f(trans_mat)), _p(radii.contiguous()), _p(_f(colors)), _p(g_m2d),
                             _p(_f(g_trans_mat)), _p(_f(g_inverse_m)), _p(_f(g_colors)), _p(_f(g_normal_opacity)),
                             _p(g_means), _p(g_scales), _p(g_rots), _p(g_opac), _p(g_shs), _p(g_rest))
    return g_means, g_scales, g_rots, g_opac, g_shs, g_rest, g_m2d


def fold_inverse_grad(trans_mat, g_inverse_m, g_trans_mat):
    """dL/dM total = g_trans_mat + adjoint(adjugate)(g_inverse_m)."""
    out = _f(g_trans_mat).clone()
    lib().orc_fold_inverse_grad(_ci(trans_mat.shape[0]), _p(_f(trans_mat)), _p(_f(g_inverse_m)), _p(out))
    return out


def _same_float(t, like):
    return t.detach().to(like.dtype).contiguous()


def cdist_top(x1, x2, largest=False, fused=True):
    """float32 or float64 (the dtype of ``x1`` decides, as in the reference's dispatch).  ``fused`` selects the
    arithmetic of the reference's CUDA build (sum = fma(t, t, sum)); False that of its CPU branch."""
    dbl = x1.dtype == torch.float64
    x1 = x1.detach().contiguous() if dbl else _f(x1)
    x2 = _same_float(x2, x1)
    N, D = x1.shape[-2], x1.shape[-1]
    M = x2.shape[-2]
    B = x1.numel() // (N * D)
    dist = torch.zeros(x1.shape[:-1], dtype=x1.dtype)
    idx = torch.zeros(x1.shape[:-1], dtype=torch.int64)
    fn = lib().orc_cdist_top_f64 if dbl else lib().orc_cdist_top
    fn(_ci(B), _ci(N), _ci(M), _ci(D), _p(x1), _p(x2), _ci(int(largest)), _ci(int(fused)), _p(dist), _p(idx))
    return dist, idx


def cdist_top_backward(x1, x2, dist, index, grad_dist):
    dbl = x1.dtype == torch.float64
    x1 = x1.detach().contiguous() if dbl else _f(x1)
    x2 = _same_float(x2, x1)
    N, D = x1.shape[-2], x1.shape[-1]
    M = x2.shape[-2]
    B = x1.numel() // (N * D)
    g1, g2 = torch.zeros_like(x1), torch.zeros_like(x2)
    fn = lib().orc_cdist_top_bwd_f64 if dbl else lib().orc_cdist_top_bwd
    fn(_ci(B), _ci(N), _ci(M), _ci(D), _p(x1), _p(x2), _p(_same_float(dist, x1)), _p(index.contiguous()),
       _p(_same_float(grad_dist, x1)), _p(g1), _p(g2))
    return g1, g2


def knn(x, c, K):
    x, c = _f(x), _f(c)
    N, D = x.shape
    M = c.shape[0]
    d2 = torch.zeros(N, K)
    idx = torch.zeros(N, K, dtype=torch.int64)
    lib().orc_knn(_ci(N), _ci(M), _ci(D), _ci(K), _p(x), _p(c), _p(d2), _p(idx))
    return d2, idx


def adam(param, grad, exp_avg, exp_avg_sq, visible, lr, b1, b2, eps, N, M):
    """In place, like ``AdamMasksedUpdated``."""
    vis = visible.to(torch.uint8).contiguous()
    lib().orc_adam(_p(param), _p(_f(grad)), _p(exp_avg), _p(exp_avg_sq), _p(vis), _cf(lr), _cf(b1), _cf(b2), _cf(eps),
                   ctypes.c_int64(N), ctypes.c_int64(M))


# ----------------------------------------------------------------------------------------------------------------
# LBS warp (fast_2d_gs/network.py:545-573, 630-645).  The reference evaluates it with lietorch.SE3 (third party,
# unpinned, absent from the reference tree): SE3.act(p) = R(q) p + t with unit quaternion (x, y, z, w).  Restated
# here with plain torch ops so autograd supplies the gradients.  Parity unpinned for this block.
# ----------------------------------------------------------------------------------------------------------------

def quat_rotate(q, p):
    """Rotate points p[...,3] by unit quaternions q[...,4] (x,y,z,w)."""
    x, y, z, w = q.unbind(-1)
    R = torch.stack([
        1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (y * w + x * z),
        2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
        2 * (x * z - y * w), 2 * (x * w + y * z), 1 - 2 * (x * x + y * y)], dim=-1).reshape(*q.shape[:-1], 3, 3)
    return (R @ p[..., None])[..., 0]


def lbs_warp(xyz, scaling_raw, rotation_raw, knn_idx, knn_w, sp_q, sp_t, sp_dr, sp_ds):
    """Rigid LBS blend: sp_q [M,4] unit quaternions, sp_t [M,3] translations (already re-centred for 'LBS_c'),
    sp_dr [M,4] additive rotation deltas, sp_ds [M,2] additive scale deltas.
    Returns warped (means, scales, rotations) as network.py:630-645 hands them to the renderer."""
    q = sp_q[knn_idx]            # [P,K,4]
    t = sp_t[knn_idx]            # [P,K,3]
    moved = quat_rotate(q, xyz[:, None, :].expand(-1, knn_idx.shape[1], -1)) + t
    d_xyz = (moved * knn_w[..., None]).sum(dim=1) - xyz
    d_rot = (sp_dr[knn_idx] * knn_w[..., None]).sum(dim=1)
    d_scale = (sp_ds[knn_idx] * knn_w[..., None]).sum(dim=1)
    means = xyz + d_xyz
    scales = torch.exp(scaling_raw) + d_scale
    rots = torch.nn.functional.normalize(rotation_raw + d_rot, dim=-1)
    return means, scales, rots


def ssim_forward(img1, img2, C1=0.01 ** 2, C2=0.03 ** 2):
    """[..., H, W] images -> (ssim_map, dm_dmu1, dm_dsigma1_sq, dm_dsigma12), 11x11 Gaussian window, zero padding."""
    x, y = _f(img1), _f(img2)
    H, W = x.shape[-2:]
    planes = x.numel() // (H * W)
    outs = [torch.zeros_like(x) for _ in range(4)]
    lib().orc_ssim_forward(_ci(planes), _ci(H), _ci(W), ctypes.c_float(C1), ctypes.c_float(C2), _p(x), _p(y),
                           _p(outs[0]), _p(outs[1]), _p(outs[2]), _p(outs[3]))
    return tuple(outs)


def ssim_backward(img1, img2, g_map, d_mu1, d_s11, d_s12):
    x, y = _f(img1), _f(img2)
    H, W = x.shape[-2:]
    planes = x.numel() // (H * W)
    out = torch.zeros_like(x)
    lib().orc_ssim_backward(_ci(planes), _ci(H), _ci(W), _p(x), _p(y), _p(_f(g_map)), _p(_f(d_mu1)), _p(_f(d_s11)),
                            _p(_f(d_s12)), _p(out))
    return out


def l1_ssim_loss(image, target, lambda_l1=0.8, lambda_ssim=0.2):
    """-> (loss, dL/dimage) of lambda_l1 * mean|image - target| + lambda_ssim * (1 - mean ssim)."""
    m, d1, d2, d3 = ssim_forward(image, target)
    n = image.numel()
    loss = lambda_l1 * (image - target).abs().mean() + lambda_ssim * (1 - m.mean())
    g = ssim_backward(image, target, torch.full_like(m, -lambda_ssim / n), d1, d2, d3)
    g = g + lambda_l1 / n * torch.sign(image - target)
    return loss, g
