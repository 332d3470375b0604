"""CPU restatement (plain torch, fp32) of the per-step superpoint motion.  TEST INFRASTRUCTURE ONLY.

Follows fast_2d_gs/network.py:1748-1776 (SC_GS_DeformNetwork.forward), freq_encoder.py:62-110 / freqencoder.cu:8-32
(encoding layout), network.py:545-549 (quaternion normalisation, translation re-centred on the superpoint) and
network.py:506-513 (kernel-weighted LBS weights).  Pinned by tests/golden/motion_w64.npz, which the reference's own
module produced.  Parameters come as a dict in torch.nn.Linear orientation (``linear.i.weight`` [out, in] ...), the
heads as ``gaussian_warp / gaussian_scaling / gaussian_rotation / local_rotation``.
"""
import torch


def freq_encode(x, degree, scale=1.0):
    """[..., D] -> [..., D * (2 * degree + 1)]: x, then sin(2^d s x), cos(2^d s x) for d = 0 .. degree-1."""
    out = [x]
    for d in range(degree):
        out += [torch.sin(x * scale * 2.0 ** d), torch.cos(x * scale * 2.0 ** d)]
    return torch.cat(out, dim=-1)


def quat_to_matrix(q):
    x, y, z, w = q.unbind(-1)
    return torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (y * w + x * z),
                        2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                        2 * (x * z - y * w), 2 * (x * w + y * z), 1 - 2 * (x * x + y * y)], dim=-1).reshape(-1, 3, 3)


def motion(points, t, sd, depth=8, skip=4, deg_p=10, deg_t=6, local_frame=True):
    """-> dict sp_q, sp_t, sp_dr, sp_ds.  ``sd``: parameter dict; ``timenet.*`` absent means no time network."""
    lin = torch.nn.functional.linear
    x_emb = freq_encode(points, deg_p)
    t_emb = freq_encode(t.view(1, 1), deg_t)
    if "timenet.0.weight" in sd:
        t_emb = lin(torch.relu(lin(t_emb, sd["timenet.0.weight"], sd["timenet.0.bias"])), sd["timenet.2.weight"],
                    sd["timenet.2.bias"])
    t_emb = t_emb.expand(points.shape[0], -1)
    h = torch.cat([x_emb, t_emb], dim=-1)
    for i in range(depth):
        h = torch.relu(lin(h, sd[f"linear.{i}.weight"], sd[f"linear.{i}.bias"]))
        if i == skip:
            h = torch.cat([x_emb, t_emb, h], dim=-1)
    d_xyz = lin(h, sd["gaussian_warp.weight"], sd["gaussian_warp.bias"])
    scaling = lin(h, sd["gaussian_scaling.weight"], sd["gaussian_scaling.bias"])
    rotation = lin(h, sd["gaussian_rotation.weight"], sd["gaussian_rotation.bias"])
    if local_frame:
        g_rot = lin(h, sd["local_rotation.weight"], sd["local_rotation.bias"])
        q = torch.nn.functional.normalize(g_rot + g_rot.new_tensor([0.0, 0.0, 0.0, 1.0]), dim=-1)
        sp_t = d_xyz + points - (quat_to_matrix(q) @ points[..., None])[..., 0]
    else:
        q = d_xyz.new_tensor([0.0, 0.0, 0.0, 1.0]).expand(points.shape[0], 4)
        sp_t = d_xyz
    return dict(sp_q=q, sp_t=sp_t, sp_dr=rotation, sp_ds=scaling[:, :2])


def kernel_weights(d2, idx, raw_radius, raw_weight=None):
    r = torch.exp(raw_radius)[idx]
    w = torch.exp(-d2 / (2 * r ** 2))
    if raw_weight is not None:
        w = w * torch.sigmoid(raw_weight)[idx]
    w = w + 1e-7
    return w / w.sum(dim=-1, keepdim=True)
