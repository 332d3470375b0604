"""Seeded synthetic stand-ins for the scenes the reference trains on (D-NeRF: 800x800 frames, 512 superpoints,
K = 3, SH degree 3; DyNeRF at half resolution: 1352x1014).  Everything is generated on the CPU with a
``torch.Generator`` so that CPU and GPU runs see identical bits, then moved to the requested device."""
import math

import torch


def look_at(eye, at=(0.0, 0.0, 0.0)):
    """World-to-view matrix of an OpenCV-convention camera (+z forward, +y down) at ``eye`` looking at ``at``.
    Same construction as the reference's ``utils/ops_3d/coord_trans_opencv.py:87-119``."""
    eye = torch.as_tensor(eye, dtype=torch.float32)
    at = torch.as_tensor(at, dtype=torch.float32)
    fwd = torch.nn.functional.normalize(at - eye, dim=-1)
    up = torch.tensor([0.0, 1.0, 0.0])
    if torch.linalg.cross(fwd, torch.tensor([0.0, -1.0, 0.0])).norm() < 1e-6:
        up = torch.tensor([0.0, 0.0, -1.0])
    right = -torch.nn.functional.normalize(torch.linalg.cross(up, fwd), dim=-1)
    down = torch.linalg.cross(fwd, right)
    R = torch.eye(4)
    R[0, :3], R[1, :3], R[2, :3] = right, down, fwd
    T = torch.eye(4)
    T[:3, 3] = -eye
    return (R @ T).contiguous()


def perspective(fovy, W, H, n=0.1, f=1000.0):
    """View-to-clip matrix (``coord_trans_opencv.py:203-245``); the fast path only shape-checks it."""
    m = torch.zeros(4, 4)
    y = math.tan(fovy * 0.5)
    x = y * W / H
    m[0, 0], m[1, 1], m[3, 2] = 1.0 / x, 1.0 / y, 1.0
    m[2, 2], m[2, 3] = f / (f - n), -(f * n) / (f - n)
    return m


def camera(W, H, eye=(0.0, 0.0, 4.0), fov=0.69, device="cpu"):
    Tw2v = look_at(eye)
    focal = 0.5 * W / math.tan(0.5 * fov)
    Tv2s = torch.tensor([[focal, 0, W / 2], [0, focal, H / 2], [0, 0, 1]], dtype=torch.float32)
    campos = torch.inverse(Tw2v)[:3, 3].contiguous()
    cam = dict(Tw2v=Tw2v, Tv2c=perspective(fov, W, H), Tv2s=Tv2s, campos=campos)
    return {k: v.to(device) for k, v in cam.items()}


def sphere_eye(radius, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    d = torch.nn.functional.normalize(torch.randn(3, generator=g), dim=-1)
    return tuple((d * radius).tolist())


def arc_eye(radius, k, n, half_angle_deg=30.0):
    a = math.radians(-half_angle_deg + 2 * half_angle_deg * (k / max(n - 1, 1)))
    return (radius * math.sin(a), 0.0, radius * math.cos(a))


def surfels(P, seed=0, log_scale_mean=-4.5, log_scale_std=0.5, device="cpu"):
    """means U[-1.3,1.3]^3, log-scales N(mean, std) on 2 axes, random unit quaternions, opacity sigmoid(N(0,1)),
    SH degree 3: DC N(0.5, 0.2), rest N(0, 0.05)."""
    g = torch.Generator().manual_seed(seed)
    s = dict(
        means=torch.rand(P, 3, generator=g) * 2.6 - 1.3,
        log_scales=torch.randn(P, 2, generator=g) * log_scale_std + log_scale_mean,
        rots_raw=torch.nn.functional.normalize(torch.randn(P, 4, generator=g), dim=-1),
        opac_raw=torch.randn(P, 1, generator=g),
        sh_dc=torch.randn(P, 1, 3, generator=g) * 0.2 + 0.5,
        sh_rest=torch.randn(P, 15, 3, generator=g) * 0.05,
    )
    s["scales"] = torch.exp(s["log_scales"])
    s["rots"] = s["rots_raw"]
    s["opac"] = torch.sigmoid(s["opac_raw"])
    return {k: v.to(device).contiguous() for k, v in s.items()}


def superpoints(means, M=512, seed=0):
    """M control points = a random subset of the means; per-superpoint rigid motion: axis-angle N(0, 0.05) as a unit
    quaternion (x,y,z,w), translation N(0, 0.02) re-centred on the superpoint ('LBS_c', network.py:549),
    additive rotation / scale deltas.  Everything on the CPU."""
    g = torch.Generator().manual_seed(7000 + seed)
    P = means.shape[0]
    centres = means[torch.randperm(P, generator=g)[:M]].contiguous()
    aa = torch.randn(M, 3, generator=g) * 0.05
    ang = aa.norm(dim=-1, keepdim=True).clamp_min(1e-12)
    q = torch.cat([aa / ang * torch.sin(ang / 2), torch.cos(ang / 2)], dim=-1)
    t = torch.randn(M, 3, generator=g) * 0.02
    dr = torch.randn(M, 4, generator=g) * 0.02
    ds = torch.randn(M, 2, generator=g) * 2e-4
    return dict(centres=centres, sp_q=q.contiguous(), sp_t_raw=t.contiguous(), sp_dr=dr.contiguous(),
                sp_ds=ds.contiguous())


def knn_points_c1(N=100_000, M=512, seed=0):
    """cdist_top / k-NN config: N points uniform in [-1,1]^3, M control points = random subset + N(0, 0.01) jitter."""
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(N, 3, generator=g) * 2 - 1
    idx = torch.randperm(N, generator=g)[:M]
    c = x[idx] + 0.01 * torch.randn(M, 3, generator=g)
    return x.contiguous(), c.contiguous()


CONFIGS = {
    "fwd_100k_800": dict(P=100_000, W=800, H=800, log_scale_mean=-4.5, log_scale_std=0.5),
    "train_100k_800": dict(P=100_000, W=800, H=800, log_scale_mean=-4.5, log_scale_std=0.5, M=512, K=3),
    "train_300k_800": dict(P=300_000, W=800, H=800, log_scale_mean=-4.5, log_scale_std=0.5, M=512, K=3),
    "multiview_500k_1352x1014": dict(P=500_000, W=1352, H=1014, log_scale_mean=-4.5, log_scale_std=0.5, M=512, K=3,
                                     views=16, radius=3.0),
    "stress_2m_1080p": dict(P=2_000_000, W=1920, H=1080, log_scale_mean=-5.5, log_scale_std=0.6, M=4096, K=8,
                            views=32, radius=3.0),
}
