"""``SparseGaussianAdam``: the reference's visibility-masked Adam (``fast_2d_gs/sparse_gaussian_adam.py:10-49``)
with every parameter group updated by ONE kernel launch instead of one launch per group."""
import ctypes

import torch

from . import _lib
from ._lib import lib, check
from .ops import _ptr, _stream


class SparseGaussianAdam(torch.optim.Adam):
    """Same constructor, ``set_before_step(visibility, N)`` and ``step()`` as the reference class; beta1 = 0.9 and
    beta2 = 0.999 are fixed and the bias correction is folded into the learning rate, as there.
    State layout (``step`` as a CPU float32 tensor, ``exp_avg``, ``exp_avg_sq``) is the reference's, so its
    checkpoints load."""

    def __init__(self, params, lr, eps):
        super().__init__(params=params, lr=lr, eps=eps)
        self.N = None
        self.visibility = None
        self._bias_cache = (None, None, None)

    def _bias_terms(self, step):
        """((1 - 0.999^t)^0.5, 1 - 0.9^t) as float32 tensors, computed once per distinct step count (all groups of a
        step share it) exactly as the reference's expression computes them."""
        t = float(step)
        if self._bias_cache[0] != t:
            self._bias_cache = (t, (1 - 0.999 ** step) ** 0.5, 1 - 0.9 ** step)
        return self._bias_cache[1], self._bias_cache[2]

    def set_before_step(self, visibility, N):
        self.visibility, self.N = visibility, N

    @torch.no_grad()
    def step(self, only=None):
        """``only``: an iterable of parameters; the step is then applied to those groups alone (each parameter keeps
        its own step count, so a step may be split to overlap with communication)."""
        self.step_visible(only)

    def step_visible(self, only=None):
        """The body of ``step`` as a plain method: ``torch.optim.Optimizer`` wraps ``step`` itself in profiling and
        hook layers that cost more host time than the launch; a training loop that has no use for them calls this."""
        batch = []
        only = None if only is None else {id(p) for p in only}
        for group in self.param_groups:
            assert len(group["params"]) == 1, "more than one tensor in group"
            param = group["params"][0]
            if only is not None and id(param) not in only:
                continue
            if param.grad is None or param.grad.numel() == 0:
                continue
            state = self.state[param]
            if len(state) == 0:
                state["step"] = torch.tensor(0.0, dtype=torch.float32)
                state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
                state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)
            state["step"] += 1
            s, b = self._bias_terms(state["step"])
            lr_eff = group["lr"] * s / b  # the reference's float32 tensor arithmetic, in its order
            batch.append((param, param.grad.detach(), state["exp_avg"], state["exp_avg_sq"], float(lr_eff),
                          group["eps"]))
        if not batch:
            return
        assert self.N is not None, "call set_before_step(visibility, N) before step()"
        masked_adam_step(batch, self.visibility, self.N)




class DenseAdam(torch.optim.Adam):
    """torch.optim.Adam for a few dense parameter tensors (the deformation network, the kernel weights), every tensor
    updated by the one launch that updates the Gaussians' tensors (``fsgs_adam_masked_multi``: each tensor is one
    "row" of its own length behind a one-element gate).  torch's fused Adam takes 0.08 ms for the 2 MB of the
    deformation network; this takes 0.005.  Same state layout as torch's (``step``, ``exp_avg``, ``exp_avg_sq``), same
    update -- ``p -= lr / (1 - b1^t) * m / (sqrt(v) / sqrt(1 - b2^t) + eps)`` -- written as the kernel's
    ``p -= lr' m / (sqrt(v) + eps')`` with ``lr' = lr sqrt(1 - b2^t) / (1 - b1^t)``, ``eps' = eps sqrt(1 - b2^t)``.
    The kernel forms ``1 - beta`` in float32, torch in double: second moments agree to 1.3e-5 relative, steps to 1e-5.
    ``step(gate=...)``: a one-element float32 device tensor; the step is applied where it is > 0 (default: applied)."""

    def __init__(self, params, lr, eps=1e-8, betas=(0.9, 0.999)):
        super().__init__(params=params, lr=lr, eps=eps, betas=betas)
        self._one = None

    @torch.no_grad()
    def step(self, gate=None):
        self.step_gated(gate)

    def step_gated(self, gate=None):
        for group in self.param_groups:
            b1, b2 = group["betas"]
            batch = []
            for param in group["params"]:
                if param.grad is None or param.numel() == 0:
                    continue
                state = self.state[param]
                if len(state) == 0:
                    state["step"] = torch.tensor(0.0, dtype=torch.float32)
                    state["exp_avg"] = torch.zeros_like(param, memory_format=torch.preserve_format)
                    state["exp_avg_sq"] = torch.zeros_like(param, memory_format=torch.preserve_format)
                state["step"] += 1
                t = float(state["step"])
                root = (1.0 - b2 ** t) ** 0.5
                batch.append((param, param.grad.detach(), state["exp_avg"], state["exp_avg_sq"],
                              group["lr"] * root / (1.0 - b1 ** t), group["eps"] * root))
            if not batch:
                continue
            if gate is None:
                if self._one is None or self._one.device != batch[0][0].device:
                    self._one = torch.ones(1, device=batch[0][0].device)
                gate = self._one
            masked_adam_step(batch, gate, 1, b1=b1, b2=b2)


def masked_adam_step(batch, visibility, N, b1=0.9, b2=0.999):
    """``batch``: list of (param, grad, exp_avg, exp_avg_sq, lr_eff, eps) with ``param.numel() % N == 0``.
    Launches ``fsgs_adam_masked_multi`` once per eight tensors."""
    vis = visibility.contiguous()
    # a float mask (visible where > 0) is the form in which the mask comes out of the gradient all-reduce
    launch = lib().fsgs_adam_masked_multi_fmask if vis.dtype == torch.float32 else lib().fsgs_adam_masked_multi
    if vis.dtype != torch.float32 and vis.dtype != torch.uint8:
        vis = vis.to(torch.uint8) if vis.dtype != torch.bool else vis
    for i in range(0, len(batch), 8):
        chunk = batch[i:i + 8]
        arr = (_lib.AdamTensor * len(chunk))()
        keep = []
        for k, (p, g, m, v, lr, eps) in enumerate(chunk):
            assert p.is_cuda and p.is_contiguous() and p.dtype == torch.float32
            g = g.contiguous()
            keep.append(g)
            arr[k].param, arr[k].grad, arr[k].exp_avg, arr[k].exp_avg_sq = p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr()
            arr[k].M, arr[k].lr, arr[k].eps = p.numel() // N, lr, eps
        check(launch(len(chunk), arr, _ptr(vis), int(N), b1, b2, _stream()), "fsgs_adam_masked_multi")
