"""Device-resident training views: the two C-ABI calls ``fsgs_view_forward`` / ``fsgs_view_backward`` behind a small
Python object that owns the workspace, the output images and the tile-list capacity of one scene.

One view of the reference's training loop (``fast_2d_gs/network.py:683-745`` and the backward autograd derives from
it) costs two crossings into ``libfsgs.so`` here -- no autograd graph, no per-step allocation, no elementwise
PyTorch kernels -- and the gradients of several views are summed in place by the kernels themselves.
"""
import ctypes

import torch

from . import _lib
from ._lib import check, lib
from .ops import _need, _ptr, _stream
from .renderer import make_lbs


class ViewEngine:
    """Buffers and capacity policy for rendering / back-propagating views of P Gaussians at W x H.

    ``forward`` fills ``images [3,H,W]``, ``opacity [H,W]``, ``extras [8,H,W]``, ``n_contrib [2,H,W]`` and ``radii [P]``
    (owned by the engine, overwritten by the next view); ``backward`` writes or accumulates the leaf gradients into
    the tensors the caller names.  The tile-list capacity starts at ``max(2^16, 8 P)`` entries and follows 1.5x the
    largest pair count seen; counters are read back asynchronously, and a view whose pairs did not fit makes the next
    ``forward`` (or ``check()``) raise after the capacity has been raised."""

    def __init__(self, P, W, H, K, M, device, sh_degree=3, n_dc=1, n_rest=15, near=0.2, far=100.0, growth=1.5):
        self.P, self.W, self.H, self.K, self.M = int(P), int(W), int(H), int(K), int(M)
        self.device = torch.device(device)
        self.sh_degree, self.n_dc, self.n_rest = sh_degree, n_dc, n_rest
        self.near, self.far, self.growth = float(near), float(far), growth
        f32 = dict(device=self.device, dtype=torch.float32)
        i32 = dict(device=self.device, dtype=torch.int32)
        self.images = torch.zeros(3, H, W, **f32)
        self.opacity = torch.zeros(H, W, **f32)
        self.extras = torch.zeros(8, H, W, **f32)
        self.n_contrib = torch.zeros(2, H, W, **i32)
        self.radii = torch.zeros(max(P, 1), **i32)[:P]
        self.counters = torch.zeros(_COUNTERS, device=self.device, dtype=torch.int64)
        self.viewspace_grad = torch.zeros(max(P, 1), 2, **f32)[:P]
        self.capacity = 0
        self.workspace = None
        self.high_water = self.last_pairs = self.overflowed = 0
        self._pending, self._free = [], []  # (event, pinned counters) in flight / reusable
        self._args = _lib.ViewArgs()
        self._lbs = None
        self._keep = None
        self._zero_opacity = None
        self._reserve(max(1 << 16, 8 * self.P))

    # ---- capacity -----------------------------------------------------------------------------------------------
    def _reserve(self, capacity):
        self.capacity = int(capacity)
        n = int(lib().fsgs_view_workspace_bytes(self.P, self.W, self.H, self.capacity, self.K, self.M))
        self.workspace = None  # release before the larger block is requested
        self.workspace = torch.empty(n, device=self.device, dtype=torch.uint8)

    def _poll(self, wait=False):
        keep = []
        for ev, host in self._pending:
            if wait:
                ev.synchronize()
            if ev.query():
                pairs = int(host[1])
                self.last_pairs = pairs
                self.high_water = max(self.high_water, pairs)
                self.overflowed += int(host[2]) > 0
                self._free.append((ev, host))
            else:
                keep.append((ev, host))
        self._pending = keep

    def check(self, wait=True):
        """Raise if an earlier view's tile lists did not fit (that view, and any step built on it, is invalid)."""
        self._poll(wait)
        if int(self.high_water * self.growth) > self.capacity:
            self._reserve(int(self.high_water * self.growth))
        if self.overflowed:
            n, self.overflowed = self.overflowed, 0
            raise RuntimeError(f"fsgs: tile lists overflowed their buffer on {n} earlier view(s); those views are "
                               "invalid (a training step that used them was dropped by the optimiser).  The "
                               "capacity has been raised; run them again.")

    # ---- one view -----------------------------------------------------------------------------------------------
    def _fill(self, scene, cam, motion):
        a = self._args
        a.P, a.W, a.H, a.sh_degree, a.n_dc, a.n_rest = self.P, self.W, self.H, self.sh_degree, self.n_dc, self.n_rest
        a.near_n, a.far_n = self.near, self.far
        a.opacity_raw, a.sh_dc, a.sh_rest = scene.opacity.data_ptr(), scene.sh_dc.data_ptr(), scene.sh_rest.data_ptr()
        ts = (scene.xyz, scene.scaling, scene.rotation, scene.knn_idx, scene.knn_w, motion["sp_q"], motion["sp_t"],
              motion["sp_dr"], motion["sp_ds"])
        self._lbs = make_lbs(*ts, pairs=getattr(scene.knn_idx, "superpoint_pairs", None))
        a.lbs = ctypes.pointer(self._lbs)
        Tw2v, Tv2s, campos = cam["Tw2v"], cam["Tv2s"], cam["campos"]
        for t in (Tw2v, Tv2s, campos):
            _need(t.is_cuda and t.is_contiguous() and t.dtype == torch.float32, "camera tensors: contiguous float32 CUDA")
        a.Tw2v, a.Tv2s, a.campos = Tw2v.data_ptr(), Tv2s.data_ptr(), campos.data_ptr()
        a.out_color, a.out_opacity, a.out_extras = self.images.data_ptr(), self.opacity.data_ptr(), self.extras.data_ptr()
        a.n_contrib, a.radii, a.counters = self.n_contrib.data_ptr(), self.radii.data_ptr(), self.counters.data_ptr()
        a.viewspace_grad = self.viewspace_grad.data_ptr()
        a.list_capacity = self.capacity
        a.workspace, a.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        self._keep = (ts, Tw2v, Tv2s, campos)  # alive until the launches have been queued and the next view starts

    def forward(self, scene, cam, motion):
        """Queue the forward of one view.  ``cam``: dict with ``Tw2v [4,4]``, ``Tv2s [3,3]``, ``campos [3]``; ``motion``:
        dict ``sp_q, sp_t, sp_dr, sp_ds`` (this view's superpoint motion).  Returns the engine (its image buffers)."""
        self.check(wait=False)
        self._fill(scene, cam, motion)
        check(lib().fsgs_view_forward(ctypes.byref(self._args), _stream()), "fsgs_view_forward")
        ev, host = self._free.pop() if self._free else (torch.cuda.Event(), torch.empty(_COUNTERS, dtype=torch.int64,
                                                                                        pin_memory=True))
        host.copy_(self.counters, non_blocking=True)
        ev.record()
        self._pending.append((ev, host))
        return self

    def backward(self, g_images, g_opacity, g_extras, grads, accumulate=False, phase=0, sh_source=None):
        """Queue the backward of the view last passed to ``forward``.  ``g_images [3,H,W]``; ``g_opacity [H,W]`` or
        None; ``g_extras [8,H,W]`` or None.  ``grads``: dict of destination tensors ``xyz, scaling, rotation, opacity,
        sh_dc, sh_rest`` and optionally ``knn_w, sp_q, sp_t, sp_dr, sp_ds, visible``.  ``phase`` 1 stops after the
        preprocess adjoint (SH and opacity gradients and the mask are then final), 2 runs the rest (LBS adjoint);
        3 stops after the compositing adjoint and writes ``sh_source`` and the mask from what is known by then, 4 runs
        the rest after 3 (preprocess and LBS adjoints).
        ``sh_source [P,7]``: receives the two factors of this view's SH gradient (clamped colour gradient, view
        direction) and its visibility; ``grads["sh_dc"]`` / ``grads["sh_rest"]`` may then be None (``ops.sh_grad_from_views``)."""
        a = self._args
        if g_extras is not None and g_opacity is None:  # the adjoint with auxiliary channels reads an opacity gradient
            if self._zero_opacity is None:
                self._zero_opacity = torch.zeros_like(self.opacity)
            g_opacity = self._zero_opacity
        for t in (g_images, g_opacity, g_extras):
            _need(t is None or (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32),
                  "upstream gradients: contiguous float32 CUDA tensors")
        a.dL_dcolor, a.dL_dopacity, a.dL_dextras = _ptr(g_images).value or 0, _ptr(g_opacity).value or 0, _ptr(g_extras).value or 0
        p = lambda name: 0 if grads.get(name) is None else grads[name].data_ptr()
        a.g_xyz, a.g_scaling_raw, a.g_rotation_raw = p("xyz"), p("scaling"), p("rotation")
        a.g_opacity_raw, a.g_sh_dc, a.g_sh_rest = p("opacity"), p("sh_dc"), p("sh_rest")
        a.g_knn_w, a.g_sp_q, a.g_sp_t, a.g_sp_dr, a.g_sp_ds = p("knn_w"), p("sp_q"), p("sp_t"), p("sp_dr"), p("sp_ds")
        a.visible = p("visible")
        a.g_sh_source = 0 if sh_source is None else sh_source.data_ptr()
        a.accumulate, a.phase = int(bool(accumulate)), int(phase)
        check(lib().fsgs_view_backward(ctypes.byref(a), _stream()), "fsgs_view_backward")


_COUNTERS = 4
