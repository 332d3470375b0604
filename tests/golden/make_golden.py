"""Generate golden vectors from the REFERENCE's own code, on CPU.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py [--ref <reference checkout>] [--only sh|ssim]

It imports the reference's PyTorch twins of the hot path (third-party packages the reference imports
but this image lacks are replaced by inert stand-ins) and, when ``oracle/_ref`` holds the compiled
reference kernels, the CPU branch of the reference's ``cdist_top``.  Outputs: small ``.npz`` files next
to this script.  The fixtures, not the reference, travel with the repository.

What each fixture pins (paths inside the reference project):
  transmat.npz    fast_compuate_transmat                renderer/gs_2d_fast_render.py:779-789  (+ autograd)
  preprocess.npz  _GS_2D_fast_preprocess_py lines 86-205 (binning patched out: it is broken as shipped,
                  :303/:318) incl. SH colours via utils/ops_3d/spherical_harmonics.py:242-302 (+ autograd)
  rasterize.npz   GS_2D_fast_rasterize (python)         renderer/gs_2d_fast_render.py:433-555  (+ autograd)
  cdist_top.npz   cdist_top / cdist_top_backward CPU branch  _C/src/other/cdist_top.cu:57-81,130-150
  sh_basis_deg7.npz  real SH of degrees 0..7, general definition  utils/ops_3d/spherical_harmonics.py:16-67
  ssim.npz        _ssim (python, five padded convolutions)  fast_2d_gs/losses/ssim.py:48-67  (+ autograd)
  motion_w64.npz  SC_GS_DeformNetwork (width 64) + head of warp()  fast_2d_gs/network.py:1670-1776, 545-549  (+ autograd)
  densify.npz     densify: clone, 2-D split, optimiser surgery     fast_2d_gs/gaussian_splatting.py:498-628, network.py:1156-1215
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def import_reference(ref):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import refpy
    refpy.import_reference(native=None, root=ref)
    from fast_2d_gs.renderer import gs_2d_fast_render as R
    from fast_2d_gs._C import get_python_function
    from utils import ops_3d
    return R, get_python_function, ops_3d


def camera(ops_3d, W, H, eye=(0.3, -0.4, 4.0), fov=0.69):
    Tw2v = ops_3d.opencv.look_at(torch.tensor(eye, dtype=torch.float32), torch.zeros(3))
    f = 0.5 * W / np.tan(0.5 * fov)
    Tv2s = torch.tensor([[f, 0, W / 2], [0, f, H / 2], [0, 0, 1]], dtype=torch.float32)
    campos = torch.inverse(Tw2v)[:3, 3].contiguous()
    return Tw2v.contiguous(), Tv2s, campos


def scene(P, seed, log_scale=-2.5, spread=1.3):
    g = torch.Generator().manual_seed(seed)
    means = (torch.rand(P, 3, generator=g) * 2 - 1) * spread
    scales = torch.exp(torch.randn(P, 2, generator=g) * 0.5 + log_scale)
    rots = torch.nn.functional.normalize(torch.randn(P, 4, generator=g), dim=-1)
    opac = torch.sigmoid(torch.randn(P, 1, generator=g))
    sh_dc = torch.randn(P, 1, 3, generator=g) * 0.2 + 0.5
    sh_rest = torch.randn(P, 15, 3, generator=g) * 0.05
    return means, scales, rots, opac, sh_dc, sh_rest


def npz(name, **arrs):
    out = {}
    for k, v in arrs.items():
        out[k] = v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KiB)")


def make_transmat(R, ops_3d):
    P = 96
    means, scales, rots, *_ = scene(P, 11)
    Tw2v, Tv2s, _ = camera(ops_3d, 128, 96)
    ins = [t.clone().requires_grad_() for t in (means, scales, rots)]
    M, n = R.fast_compuate_transmat(*ins, Tw2v, Tv2s)
    g = torch.Generator().manual_seed(12)
    gM, gn = torch.randn(M.shape, generator=g), torch.randn(n.shape, generator=g)
    torch.autograd.backward([M, n], [gM, gn])
    npz("transmat.npz", means=means, scales=scales, rots=rots, Tw2v=Tw2v, Tv2s=Tv2s, M=M, normal=n, gM=gM, gn=gn,
        g_means=ins[0].grad, g_scales=ins[1].grad, g_rots=ins[2].grad)


def make_preprocess(R, ops_3d):
    P, W, H = 384, 120, 90
    means, scales, rots, opac, sh_dc, sh_rest = scene(P, 21)
    means[:8, 2] = 5.0  # behind / too close to the camera: exercises the z <= 0.2 cull
    Tw2v, Tv2s, campos = camera(ops_3d, W, H)
    Tv2c = ops_3d.opencv.perspective(0.69, size=(W, H))
    R._prepare_py = lambda *a, **k: (None, None)  # broken as shipped; binning is pinned elsewhere
    ins = [t.clone().requires_grad_() for t in (means, scales, rots, opac, sh_dc, sh_rest)]
    for deg in (3, 0):
        for t in ins:
            t.grad = None
        out = R._GS_2D_fast_preprocess_py(W, H, deg, False, ins[0], ins[1], ins[2], ins[3], ins[4],
                                          ins[5] if deg > 0 else None, Tw2v, Tv2c, Tv2s, campos)
        means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii = out[:7]
        g = torch.Generator().manual_seed(22 + deg)
        ups = [torch.randn(t.shape, generator=g) for t in (means2D, colors, trans_mat, inverse_m, normal_opacity)]
        torch.autograd.backward([means2D, colors, trans_mat, inverse_m, normal_opacity], ups)
        grads = {f"g_{n}": (t.grad if t.grad is not None else torch.zeros_like(t))
                 for n, t in zip(("means", "scales", "rots", "opac", "sh_dc", "sh_rest"), ins)}
        npz(f"preprocess_deg{deg}.npz", W=W, H=H, deg=deg, means=means, scales=scales, rots=rots, opac=opac,
            sh_dc=sh_dc, sh_rest=sh_rest, Tw2v=Tw2v, Tv2s=Tv2s, campos=campos, means2D=means2D, colors=colors,
            trans_mat=trans_mat, inverse_m=inverse_m, normal_opacity=normal_opacity, depths=depths, radii=radii,
            up_means2D=ups[0], up_colors=ups[1], up_trans_mat=ups[2], up_inverse_m=ups[3], up_normal_opacity=ups[4],
            **grads)


def make_rasterize(R, get_python_function, ops_3d):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc  # only to obtain per-tile lists to feed the reference's python compositor
    P, W, H = 400, 72, 56
    # seed chosen so that no splat sits on the alpha = 1/255 cut for any pixel: there the twin (cross products of
    # trans_mat rows) and the CUDA formulation (inverse_m rows) may round to different sides
    means, scales, rots, opac, sh_dc, sh_rest = scene(P, 32, log_scale=-1.6)
    Tw2v, Tv2s, campos = camera(ops_3d, W, H)
    pre = orc.preprocess_forward(W, H, 3, means, scales, rots, opac, sh_dc, sh_rest, Tw2v, Tv2s, campos)
    means2D, colors, trans_mat, inverse_m, normal_opacity, depths, radii, ranges, point_list = pre[:9]
    n_real = pre[10]
    point_list = point_list[:n_real].contiguous()
    rast = R.GS_2D_fast_rasterize  # without a compiled extension the decorator leaves the python twin in place
    ins = [t.clone().requires_grad_() for t in (means2D, colors, normal_opacity, trans_mat)]
    images, opacities, extras, n_contrib = rast(W, H, ins[0], ins[1], ins[2], ins[3], inverse_m, ranges,
                                                point_list.long(), 0.2, 100., False)
    g = torch.Generator().manual_seed(32)
    g_img, g_op = torch.randn(images.shape, generator=g), torch.randn(opacities.shape, generator=g)
    g_nrm = torch.randn(3, H, W, generator=g)
    torch.autograd.backward([images, opacities, extras[1:4]], [g_img, g_op, g_nrm])
    npz("rasterize.npz", W=W, H=H, means2D=means2D, colors=colors, normal_opacity=normal_opacity,
        trans_mat=trans_mat, inverse_m=inverse_m, ranges=ranges, point_list=point_list, images=images,
        opacities=opacities, extras=extras, n_contrib=n_contrib, g_img=g_img, g_op=g_op, g_nrm=g_nrm,
        g_means2D=ins[0].grad, g_colors=ins[1].grad, g_normal_opacity=ins[2].grad, g_trans_mat=ins[3].grad)


def make_sh_basis():
    """Real SH of degrees 0..7 at random unit directions by the reference's general definition."""
    from utils.ops_3d import spherical_harmonics as S
    g = torch.Generator().manual_seed(41)
    d = torch.nn.functional.normalize(torch.randn(48, 3, generator=g, dtype=torch.float64), dim=-1)
    theta, phi = torch.acos(d[:, 2].clamp(-1, 1)), torch.atan2(d[:, 1], d[:, 0])
    Y = torch.stack([S._SH(l, m, theta, phi) for l in range(8) for m in range(-l, l + 1)], dim=-1)
    npz("sh_basis_deg7.npz", dirs=d.float(), Y=Y.float())


def make_ssim(get_python_function):
    """SSIM map of the reference's python ``_ssim`` (losses/ssim.py:48-67) and its autograd gradient."""
    from fast_2d_gs.losses import ssim as S
    g = torch.Generator().manual_seed(51)
    a = torch.rand(2, 3, 37, 45, generator=g)
    b = (a + 0.2 * torch.randn(2, 3, 37, 45, generator=g)).clamp(0, 1)
    a.requires_grad_()
    window = S.create_window(11, 3)
    m = S._ssim(a, b, window)  # the python twin: the compiled operators are absent in this container
    up = torch.randn(m.shape, generator=g)
    m.backward(up)
    npz("ssim.npz", img1=a, img2=b, ssim_map=m, up=up, g_img1=a.grad)


def make_cdist_top():
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    sys.path.insert(0, ref_dir)
    try:
        import _C as refC
    except ImportError as e:
        print(f"oracle/_ref not built ({e}); cdist_top.npz not regenerated")
        return
    g = torch.Generator().manual_seed(41)
    x = torch.rand(2, 700, 3, generator=g) * 2 - 1
    c = torch.rand(2, 48, 3, generator=g) * 2 - 1
    c[:, 5] = c[:, 17]  # exact duplicates: exercises the tie rule
    c[:, 30] = c[:, 17]
    out = {}
    for largest in (False, True):
        d, i = refC.cdist_top(x, c, largest)
        gd = torch.randn(d.shape, generator=g)
        g1, g2 = refC.cdist_top_backward(x, c, d, i, gd)
        tag = "far" if largest else "near"
        out.update({f"dist_{tag}": d, f"idx_{tag}": i, f"gd_{tag}": gd, f"g1_{tag}": g1, f"g2_{tag}": g2})
    x5 = torch.randn(300, 5, generator=g)
    c5 = torch.randn(20, 5, generator=g)
    d5, i5 = refC.cdist_top(x5, c5, False)
    npz("cdist_top.npz", x=x, c=c, x5=x5, c5=c5, dist5=d5, idx5=i5, **out)


def quat_to_matrix(q):
    x, y, z, w = q.unbind(-1)
    return torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (y * w + x * z),
                        2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                        2 * (x * z - y * w), 2 * (x * w + y * z), 1 - 2 * (x * x + y * y)], dim=-1).reshape(-1, 3, 3)


def make_motion():
    """The reference's deformation network (SC_GS_DeformNetwork, network.py:1670-1776) at width 64 with its fourth
    head, evaluated on 37 superpoint centres at one time, followed by the head of warp() (network.py:545-549;
    lietorch's SO3.act restated as a rotation matrix), and the autograd gradients of every parameter for random
    upstream gradients on the four motion tensors.  The frequency encoder is the reference's PyTorch twin
    (freq_encoder.py:62-110): its compiled one (freqencoder.cu) needs a GPU and produces the same layout."""
    from fast_2d_gs import network as N
    from fast_2d_gs.freq_encoder import FreqEncoder_torch
    N.FreqEncoder = FreqEncoder_torch
    torch.manual_seed(61)
    net = N.SC_GS_DeformNetwork(D=8, W=64, pos_enc_p_cfg=dict(degree=10), pos_enc_t_cfg=dict(degree=6),
                                is_blender=True, local_frame=True)
    g = torch.Generator().manual_seed(62)
    with torch.no_grad():  # heads that move something (the reference starts them at 1e-5)
        for head, std in ((net.gaussian_warp, 0.05), (net.gaussian_scaling, 0.02), (net.gaussian_rotation, 0.05),
                          (net.local_rotation, 0.3)):
            head.weight.copy_(torch.randn(head.weight.shape, generator=g) * std)
            head.bias.copy_(torch.randn(head.bias.shape, generator=g) * std)
        for layer in net.linear:
            layer.bias.copy_(torch.randn(layer.bias.shape, generator=g) * 0.1)
    M = 37
    c = torch.rand(M, 3, generator=g) * 2 - 1
    t = torch.tensor([0.37])
    d_xyz, rotation, scaling, local_rot = net(c, t)
    q = torch.nn.functional.normalize(local_rot + torch.tensor([0.0, 0.0, 0.0, 1.0]), dim=-1)
    sp_t = d_xyz + c - (quat_to_matrix(q) @ c[..., None])[..., 0]
    outs = dict(sp_q=q, sp_t=sp_t, sp_dr=rotation, sp_ds=scaling[:, :2])
    ups = {k: torch.randn(v.shape, generator=g) for k, v in outs.items()}
    torch.autograd.backward([outs[k] for k in outs], [ups[k] for k in outs])
    arrs = dict(points=c, t=t)
    arrs.update({"out_" + k: v for k, v in outs.items()})
    arrs.update({"up_" + k: v for k, v in ups.items()})
    for name, p in net.named_parameters():
        arrs["param_" + name] = p.detach()
        arrs["grad_" + name] = p.grad
    npz("motion_w64.npz", **arrs)


def make_densify():
    """The reference's own ``densify`` (gaussian_splatting.py:623-628 -> densify_and_clone :608-622, the 2-D
    densify_and_split of network.py:1156-1185, densification_postfix, prune_points, change_optimizer :498-548) run on
    a bare instance of its model class with 300 Gaussians, an Adam optimiser that has taken steps, and gathered
    statistics.  ``torch.normal`` is replaced for the call by mean + std * z with stored draws z, so that the split
    children are reproducible."""
    from fast_2d_gs import network as N
    g = torch.Generator().manual_seed(71)
    P = 300
    m = object.__new__(N.FastSuperpoint2DGaussianSplatting)
    torch.nn.Module.__init__(m)
    vals = dict(_xyz=torch.rand(P, 3, generator=g) * 2 - 1, _features_dc=torch.randn(P, 1, 3, generator=g),
                _features_rest=torch.randn(P, 15, 3, generator=g) * 0.1,
                _scaling=torch.randn(P, 2, generator=g) * 0.7 - 3.0, _rotation=torch.randn(P, 4, generator=g),
                _opacity=torch.randn(P, 1, generator=g))
    for k, v in vals.items():
        setattr(m, k, torch.nn.Parameter(v.clone()))
    m._step, m.stages, m.init_same_scale = 0, {"sp_fix": (0, 0, 0)}, "none"
    m.scaling_activation, m.scaling_activation_inverse = torch.exp, torch.log
    m.adaptive_control_cfg, m.render_method, m.use_so3, m.p2sp = {"blur_split": False}, "2d_gs_fast", False, None
    m._culling, m.factor_culling = torch.zeros(P, 1, dtype=torch.bool), torch.ones(P, 1)
    m.xyz_gradient_accum = (torch.rand(P, 1, generator=g) ** 3) * 1e-3 * 40
    m.denom = torch.randint(0, 40, (P, 1), generator=g).float()   # zeros among them: grads NaN -> 0
    m.max_radii2D = torch.zeros(P)
    groups = [dict(params=[getattr(m, a)], lr=1e-3, name=n) for a, n in m.param_names_map.items()]
    opt = torch.optim.Adam(groups, lr=0.0, eps=1e-15)
    for _ in range(2):
        for a in m.param_names_map:
            p = getattr(m, a)
            p.grad = torch.randn(p.shape, generator=g)
        opt.step()
    before = {a: getattr(m, a).detach().clone() for a in m.param_names_map}
    state = {a: (opt.state[getattr(m, a)]["exp_avg"].clone(), opt.state[getattr(m, a)]["exp_avg_sq"].clone())
             for a in m.param_names_map}
    accum, denom = m.xyz_gradient_accum.clone(), m.denom.clone()
    z = torch.randn(4 * P, 3, generator=g)
    real_normal = torch.normal
    torch.normal = lambda mean, std: mean + std * z[:mean.shape[0]]
    try:
        with torch.no_grad():
            m.densify(opt, 2e-4, 4.0, 0.01)
    finally:
        torch.normal = real_normal
    arrs = dict(max_grad=2e-4, extent=4.0, percent_dense=0.01, accum=accum, denom=denom, z=z)
    for a in m.param_names_map:
        p = getattr(m, a)
        arrs["in" + a], arrs["out" + a] = before[a], p.detach()
        arrs["in_m" + a], arrs["in_v" + a] = state[a]
        arrs["out_m" + a], arrs["out_v" + a] = opt.state[p]["exp_avg"], opt.state[p]["exp_avg_sq"]
    npz("densify.npz", **arrs)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None, help="reference checkout (default: $FSGS_REFERENCE_ROOT, else a "
                                                "directory named 'reference' beside this repository)")
    ap.add_argument("--only", default=None, help="\"sh\" / \"ssim\" / \"motion\": regenerate that fixture alone")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from refpath import reference_root
    args.ref = reference_root(args.ref)
    if args.ref is None:
        raise SystemExit("reference checkout not found: pass --ref or set FSGS_REFERENCE_ROOT")
    torch.set_num_threads(4)
    if args.only == "sh":
        import_reference(args.ref)
        make_sh_basis()
        return
    if args.only == "ssim":
        make_ssim(import_reference(args.ref)[1])
        return
    if args.only == "densify":
        import_reference(args.ref)
        make_densify()
        return
    if args.only == "motion":
        import_reference(args.ref)
        make_motion()
        return
    make_cdist_top()
    R, get_python_function, ops_3d = import_reference(args.ref)
    make_sh_basis()
    make_transmat(R, ops_3d)
    make_preprocess(R, ops_3d)
    make_rasterize(R, get_python_function, ops_3d)
    make_ssim(get_python_function)
    make_motion()
    make_densify()


if __name__ == "__main__":
    main()
