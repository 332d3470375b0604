"""Multi-GPU layer: one process per GPU, views sharded across ranks, per-Gaussian gradients summed by one
all-reduce over a flat bucket (NCCL on GPUs, gloo in the CPU tests).  The reference renders a batch of views in a
serial loop on one device (``fast_2d_gs/network.py:683-745``); every view only reads the replicated parameters,
so views are independent units and the only exchange is the gradient sum before the optimizer step.
"""
import torch
import torch.distributed as dist


def shard_views(n_views, rank, world_size):
    """Views of a batch handled by ``rank``: rank, rank + world_size, ...  (sums are taken in this order)."""
    return list(range(rank, n_views, world_size))


def slot_order(world_size, slots_per_rank):
    """All-gathered view slots in view order.  After an all-gather of ``slots_per_rank`` slots from each of
    ``world_size`` ranks, slot ``r * slots_per_rank + j`` holds rank r's j-th view, which ``shard_views`` numbers
    ``r + j * world_size``; the returned list names the slots by ascending view number (views past the end of a batch
    are empty slots and sort where their number would be)."""
    return [r * slots_per_rank + j for j in range(slots_per_rank) for r in range(world_size)]


class GradBucket:
    """A flat fp32 buffer holding the gradients of ``params`` back to back, plus ``extra`` floats that ride in the
    same collectives (the visibility mask as 0/1), placed after parameter number ``extra_after`` (default: at the
    end).  The buffer is a sequence of segments -- one per parameter, one for the extra block -- and collectives act
    on runs of segments.  ``reduce()`` copies in only the ``.grad`` tensors that do not already live in their slice
    (``view_of(p)`` handed to the backward kernels as the destination makes the copy unnecessary), all-reduces the
    whole buffer and re-points every ``.grad`` at its slice."""

    def __init__(self, params, extra=0, extra_after=None):
        self.params = list(params)
        self.sizes = [p.numel() for p in self.params]
        k = len(self.params) if extra_after is None else extra_after + 1
        seg_sizes = self.sizes[:k] + [extra] + self.sizes[k:]
        self.extra_segment = k
        # every segment starts on a 256-byte boundary whatever the row count: kernels store float2 / float4 rows into
        # these views; the padding between segments stays zero and rides along in the collectives
        pad = lambda n: (n + 63) & ~63
        self.flat = torch.zeros(sum(pad(n) for n in seg_sizes), dtype=torch.float32, device=self.params[0].device)
        self.bounds, off = [], 0
        for n in seg_sizes:
            self.bounds.append((off, off + n))
            off += pad(n)
        seg_views = [self.flat[lo:hi] for lo, hi in self.bounds]
        self.extra = seg_views[k]
        self.views = [v.view(p.shape) for v, p in zip(seg_views[:k] + seg_views[k + 1:], self.params)]
        self.copied = 0  # gradients that had to be copied in by the last pack()

    def nbytes(self):
        return self.flat.numel() * 4

    def view_of(self, param):
        for p, v in zip(self.params, self.views):
            if p is param:
                return v
        raise KeyError("parameter is not in this bucket")

    def pack(self):
        dst, src = [], []
        for p, v in zip(self.params, self.views):
            if p.grad is None:
                v.zero_()
            elif p.grad.data_ptr() != v.data_ptr():
                dst.append(v)
                src.append(p.grad)
        self.copied = len(src)
        if src:
            torch._foreach_copy_(dst, src)

    def adopt(self):
        """Point every ``.grad`` at its slice of the buffer."""
        for p, v in zip(self.params, self.views):
            p.grad = v

    def reduce(self, group=None, async_op=False):
        self.pack()
        work = None
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        self.adopt()
        return work

    def span(self, first, last):
        """Flat slice covering segments ``first`` .. ``last`` (inclusive)."""
        return self.flat[self.bounds[first][0]:self.bounds[last][1]]

    def reduce_span(self, first, last, group=None):
        """Asynchronous all-reduce of a run of segments (their contents must already be in place); returns the work
        handle, or None when there is nobody to talk to.  ``.wait()`` orders the current stream after it."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            return dist.all_reduce(self.span(first, last), op=dist.ReduceOp.SUM, group=group, async_op=True)
        return None


def reduce_visibility(visible, group=None):
    """Union of the per-rank visibility masks (bool [P]) -> bool [P] on every rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return visible
    v = visible.to(torch.uint8)
    dist.all_reduce(v, op=dist.ReduceOp.MAX, group=group)
    return v.bool()


def reduce_max_(t, group=None):
    """In-place element-wise maximum across ranks (radii, running maxima of the densification statistics)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t
