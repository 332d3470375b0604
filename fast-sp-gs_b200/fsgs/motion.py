"""The per-step superpoint motion as one operator: deformation network on the superpoint centres at time ``t``
(``SC_GS_DeformNetwork``, fast_2d_gs/network.py:1670-1776) -> unit quaternion, re-centred translation, additive
rotation and scale deltas (the head of ``warp``, network.py:545-549), and the kernel-weighted LBS weights
(``calc_LBS_weight``, network.py:506-513).  One kernel forward and two backward per evaluation instead of the
reference's chain of some seventy PyTorch launches; all parameters in one flat tensor (one optimiser launch, one
contiguous segment of the gradient exchange)."""
import ctypes
import math

import torch

from . import _lib
from ._lib import check, lib
from .ops import _need, _ptr, _stream


class MotionNet:
    """``params`` is the flat fp32 parameter tensor (a ``torch.nn.Parameter``); ``views()`` gives named views in
    ``torch.nn.Linear`` orientation for loading / saving a reference ``state_dict``."""

    def __init__(self, M, device="cuda", depth=8, width=256, skip=4, deg_p=10, deg_t=6, time_hidden=256, time_out=30,
                 local_frame=False, scale_p=1.0, scale_t=1.0, seed=None):
        c = self.cfg = _lib.MotionCfg()
        c.M, c.depth, c.width, c.skip, c.deg_p, c.deg_t = M, depth, width, skip, deg_p, deg_t
        c.time_hidden, c.time_out, c.local_frame, c.scale_p, c.scale_t = time_hidden, time_out, int(local_frame), scale_p, scale_t
        n = int(lib().fsgs_motion_param_count(ctypes.byref(c)))
        _need(n > 0, "unsupported deformation-network shape (see include/fsgs.h)")
        off = (ctypes.c_int64 * (6 + 2 * depth))()
        ins = (ctypes.c_int32 * depth)()
        check(lib().fsgs_motion_param_offsets(ctypes.byref(c), off, ins), "fsgs_motion_param_offsets")
        self.offsets, self.inputs = list(off), list(ins)
        self.device = torch.device(device)
        self.n_heads = 14 if local_frame else 10
        self.params = torch.nn.Parameter(torch.zeros(n, device=self.device))
        self.workspace = torch.empty(int(lib().fsgs_motion_workspace_bytes(ctypes.byref(c))), dtype=torch.uint8,
                                     device=self.device)
        self.reset_parameters(seed)

    # ---- parameter views ----------------------------------------------------------------------------------------
    def sections(self):
        """[(name, offset, inputs, outputs)] of every matrix (stored [inputs, outputs]) and bias (inputs = 0)."""
        c, o = self.cfg, self.offsets
        Et = 2 * c.deg_t + 1
        out = []
        if c.time_out > 0:
            out += [("timenet.0.weight", o[0], Et, c.time_hidden), ("timenet.0.bias", o[1], 0, c.time_hidden),
                    ("timenet.2.weight", o[2], c.time_hidden, c.time_out), ("timenet.2.bias", o[3], 0, c.time_out)]
        for i in range(c.depth):
            out += [(f"linear.{i}.weight", o[4 + 2 * i], self.inputs[i], c.width), (f"linear.{i}.bias", o[5 + 2 * i], 0, c.width)]
        out += [("heads.weight", o[4 + 2 * c.depth], c.width, self.n_heads), ("heads.bias", o[5 + 2 * c.depth], 0, self.n_heads)]
        return out

    def views(self, flat=None):
        flat = self.params.data if flat is None else flat
        v = {}
        for name, off, n_in, n_out in self.sections():
            v[name] = flat[off:off + max(n_in, 1) * n_out].view(n_in, n_out) if n_in else flat[off:off + n_out]
        return v

    @torch.no_grad()
    def reset_parameters(self, seed=None):
        """The reference's initialisation (network.py:1731-1746): Kaiming-uniform layers with zero bias, heads drawn
        from narrow normals (1e-5; scale 1e-8; local rotation 1e-4) with zero bias, PyTorch's default for the time
        network."""
        g = torch.Generator().manual_seed(0 if seed is None else seed)
        v = self.views()
        self.params.data.zero_()
        for name, w in v.items():
            if name.startswith("linear") and name.endswith("weight"):
                bound = math.sqrt(6.0 / w.shape[0])
                w.copy_((torch.rand(w.shape, generator=g) * 2 - 1) * bound)
            elif name.startswith("timenet"):
                fan_in = v[name.replace("bias", "weight")].shape[0]
                w.copy_((torch.rand(w.shape, generator=g) * 2 - 1) / math.sqrt(fan_in))
        h = v["heads.weight"]
        h[:, 0:3] = torch.randn(h.shape[0], 3, generator=g) * 1e-5
        h[:, 3:6] = torch.randn(h.shape[0], 3, generator=g) * 1e-8
        h[:, 6:10] = torch.randn(h.shape[0], 4, generator=g) * 1e-5
        if self.cfg.local_frame:
            h[:, 10:14] = torch.randn(h.shape[0], 4, generator=g) * 1e-4

    @torch.no_grad()
    def load_reference_state_dict(self, sd):
        """Copy a ``SC_GS_DeformNetwork.state_dict()`` in (weights transposed into [inputs, outputs])."""
        v = self.views()
        for name, w in v.items():
            if name.startswith("heads"):
                continue
            src = sd[name].to(self.device)
            w.copy_(src.t() if src.dim() == 2 else src)
        heads = ["gaussian_warp", "gaussian_scaling", "gaussian_rotation"] + (["local_rotation"] if self.cfg.local_frame else [])
        v["heads.weight"].copy_(torch.cat([sd[h + ".weight"] for h in heads], dim=0).t().to(self.device))
        v["heads.bias"].copy_(torch.cat([sd[h + ".bias"] for h in heads], dim=0).to(self.device))

    # ---- evaluation ---------------------------------------------------------------------------------------------
    def _args(self, sp_points, t):
        a = _lib.MotionArgs()
        a.cfg = self.cfg
        _need(sp_points.is_cuda and sp_points.is_contiguous() and tuple(sp_points.shape) == (self.cfg.M, 3),
              "sp_points: contiguous float32 CUDA tensor [M,3]")
        _need(t.is_cuda and t.numel() == 1 and t.dtype == torch.float32, "t: float32 CUDA tensor with one element")
        a.sp_points, a.t, a.params = sp_points.data_ptr(), t.data_ptr(), self.params.data_ptr()
        a.workspace, a.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        return a

    def forward(self, sp_points, t, out=None):
        """-> dict ``sp_q [M,4], sp_t [M,3], sp_dr [M,4], sp_ds [M,2]`` (into ``out`` when given).  The workspace keeps
        what ``backward`` needs until the next ``forward``."""
        M = self.cfg.M
        if out is None:
            f = lambda k: torch.empty(M, k, device=self.device)
            out = dict(sp_q=f(4), sp_t=f(3), sp_dr=f(4), sp_ds=f(2))
        a = self._args(sp_points, t)
        a.sp_q, a.sp_t, a.sp_dr, a.sp_ds = (out[k].data_ptr() for k in ("sp_q", "sp_t", "sp_dr", "sp_ds"))
        check(lib().fsgs_motion_forward(ctypes.byref(a), _stream()), "fsgs_motion_forward")
        self._last = (sp_points, t)
        return out

    def backward(self, grads, g_params, accumulate=False):
        """``grads``: dict ``sp_q, sp_t, sp_dr, sp_ds`` of the loss gradients of the last ``forward``'s outputs;
        ``g_params`` (flat, same layout as ``params``) is written, or added to when ``accumulate``."""
        a = self._args(*self._last)
        a.g_sp_q, a.g_sp_t, a.g_sp_dr, a.g_sp_ds = (grads[k].data_ptr() for k in ("sp_q", "sp_t", "sp_dr", "sp_ds"))
        a.g_params, a.accumulate = g_params.data_ptr(), int(bool(accumulate))
        check(lib().fsgs_motion_backward(ctypes.byref(a), _stream()), "fsgs_motion_backward")


def kernel_weights(d2, idx, raw_radius, raw_weight=None, out=None):
    """LBS weights of the shipped configuration ('weighted_kernel', network.py:506-513) in one launch."""
    P, K = d2.shape
    out = torch.empty_like(d2) if out is None else out
    check(lib().fsgs_lbs_weights_forward(P, K, _ptr(d2), _ptr(idx), _ptr(raw_radius), _ptr(raw_weight), _ptr(out),
                                         _stream()), "fsgs_lbs_weights_forward")
    return out


def kernel_weights_backward(d2, idx, raw_radius, raw_weight, g_w, pairs, g_radius, g_weight=None, accumulate=False):
    """``pairs`` = ``renderer.group_pairs_by_superpoint(idx, M)``; gradients of the raw radius / raw weight [M]."""
    P, K = d2.shape
    offsets, ids = pairs
    scratch = torch.empty(int(lib().fsgs_lbs_weights_backward_workspace_bytes(P, K)), dtype=torch.uint8, device=d2.device)
    check(lib().fsgs_lbs_weights_backward(P, K, raw_radius.shape[0], _ptr(d2), _ptr(idx), _ptr(raw_radius),
                                          _ptr(raw_weight), _ptr(g_w), _ptr(offsets), _ptr(ids), _ptr(g_radius),
                                          _ptr(g_weight), int(bool(accumulate)), _ptr(scratch), scratch.numel(),
                                          _stream()), "fsgs_lbs_weights_backward")
