"""Host logic of the multi-GPU layer on CPU: two gloo ranks share views and sum gradients through GradBucket."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, out):
    sys.path.insert(0, os.path.join(ROOT, "fast-sp-gs_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fsgs.dist import GradBucket, reduce_max_, reduce_visibility, shard_views
    views = shard_views(5, rank, world)
    g = torch.Generator().manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(7, 3, generator=g)), torch.nn.Parameter(torch.randn(7, 15, 3, generator=g)),
              torch.nn.Parameter(torch.randn(7, 1, generator=g))]
    # every view contributes a gradient that depends on the view only: the sum over ranks must equal the serial sum
    for p in params:
        p.grad = sum(torch.full_like(p, float(v + 1)) * p.detach() for v in views)
    # the second gradient is produced in place (as the backward kernels do), the others are copied in; the
    # visibility mask rides in the bucket's tail
    bucket = GradBucket(params, extra=7)
    in_place = bucket.view_of(params[1])
    in_place.copy_(params[1].grad)
    params[1].grad = in_place.detach()
    mask = torch.zeros(7, dtype=torch.bool)
    mask[rank::3] = True
    bucket.extra.copy_(mask)
    bucket.reduce()
    ok = bucket.copied == 2 and (bucket.extra > 0).tolist() == [True, True, False, True, True, False, True]
    params[2].grad = None          # a parameter without gradient contributes zeros
    bucket.reduce()
    ok &= bool((params[2].grad == 0).all())
    for p in params:
        p.grad = sum(torch.full_like(p, float(v + 1)) * p.detach() for v in views)
    bucket.reduce()
    expect = [sum(float(v + 1) for v in range(5)) * p.detach() for p in params]
    ok &= all(torch.allclose(p.grad, e, rtol=1e-6) for p, e in zip(params, expect))
    ok &= all(p.grad.data_ptr() == v.data_ptr() for p, v in zip(params, bucket.views))
    vis = torch.zeros(7, dtype=torch.bool)
    vis[rank::3] = True
    vis = reduce_visibility(vis)
    ok &= vis.tolist() == [True, True, False, True, True, False, True]
    # the split exchange of the training step: mask placed after the first parameter, two runs of segments
    split = GradBucket(params, extra=7, extra_after=0)
    for p in params:
        p.grad = None
    for p, v in zip(params, split.views):
        v.copy_(float(rank + 1) * p.detach())
        p.grad = v.detach()
    split.extra.copy_(mask)
    first = split.reduce_span(0, 1)
    split.pack()
    second = split.reduce_span(2, 3)
    first.wait()
    second.wait()
    split.adopt()
    ok &= split.copied == 0 and all(torch.allclose(p.grad, 3.0 * p.detach()) for p in params)
    ok &= (split.extra > 0).tolist() == [True, True, False, True, True, False, True]
    ok &= split.span(0, 1).numel() >= 7 * 3 + 7 and split.span(2, 3).numel() >= 7 * 45 + 7
    ok &= all(v.data_ptr() % 256 == split.flat.data_ptr() % 256 for v in split.views)   # segments keep alignment
    # the factor exchange of the training step: every rank contributes the same number of view slots (empty ones are
    # zero), an all-gather delivers them rank-major, slot_order names them in view order
    from fsgs.dist import slot_order
    slots = 3                                       # ceil(5 views / 2 ranks)
    send = torch.zeros(slots, 4, 7)
    for j, v in enumerate(views):
        send[j] = float(v + 1)                      # view number + 1; 0 marks an empty slot
    recv = torch.empty(world * slots, 4, 7)
    dist.all_gather_into_tensor(recv.view(-1), send.view(-1))
    seen = [int(recv[k, 0, 0]) for k in slot_order(world, slots)]
    ok &= seen == [1, 2, 3, 4, 5, 0]
    radii = torch.tensor([rank, 5 - rank, 2], dtype=torch.int32)
    ok &= reduce_max_(radii).tolist() == [1, 5, 2]
    out[rank] = (bool(ok), views)
    dist.destroy_process_group()


def test_two_ranks_shard_views_and_sum_gradients():
    mp.set_start_method("spawn", force=True)
    with mp.Manager() as m:
        out = m.dict()
        port = 29500 + os.getpid() % 2000
        mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
        assert out[0][0] and out[1][0]
        assert out[0][1] == [0, 2, 4] and out[1][1] == [1, 3]


def test_single_process_bucket_is_a_noop_reduce():
    sys.path.insert(0, os.path.join(ROOT, "fast-sp-gs_b200"))
    from fsgs.dist import GradBucket, reduce_visibility, shard_views
    assert shard_views(16, 3, 8) == [3, 11] and shard_views(2, 5, 8) == []
    p = torch.nn.Parameter(torch.ones(4, 2))
    p.grad = torch.full((4, 2), 3.0)
    b = GradBucket([p])
    assert b.reduce() is None and torch.equal(p.grad, torch.full((4, 2), 3.0)) and b.nbytes() >= 32
    v = torch.tensor([True, False])
    assert reduce_visibility(v) is v
