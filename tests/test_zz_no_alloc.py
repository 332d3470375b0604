"""The allocation-free binning entry point against the workspace-taking one, through the C ABI.

``fsgs_bin_tiles_noalloc`` exists for hosts that may not touch the CUDA allocator while rendering (a plug-in or
viewer handed a fixed device-memory budget at start-up; a plain C program without a caching allocator, for which
a per-frame cudaMalloc/cudaFree would stall the device).  Its scratch is a fixed array inside the library that
every call on the device shares and that keeps whatever the previous call left behind, so the test calls it
twice in a row -- on two different scenes -- and wants tile ranges and tile lists identical, element for
element, to what ``fsgs_bin_tiles`` produces from the same inputs (integer outputs: no tolerance).
This file sorts last on purpose: a run that stops at the first failure has by then run every other test.
"""
import ctypes

import pytest
import torch

from util import make_scene

pytestmark = pytest.mark.gpu


def _bin(entry, W, H, o, opac, capacity, with_workspace):
    from fsgs import _lib, ops
    dev = opac.device
    T = ((W + 15) // 16) * ((H + 15) // 16)
    ranges = torch.full((T, 2), -7, device=dev, dtype=torch.int64)
    point_list = torch.full((capacity,), -7, device=dev, dtype=torch.int32)
    tile_order = torch.full((T,), -7, device=dev, dtype=torch.int32)
    b = _lib.BinArgs()
    b.P, b.W, b.H = opac.shape[0], W, H
    p = ops._ptr
    b.means2D, b.inverse_m, b.depths, b.opac = p(o["means2D"]), p(o["inverse_m"]), p(o["depths"]), p(opac)
    b.radii, b.tile_counts, b.counters = p(o["radii"]), p(o["tile_counts"]), p(o["counters"])
    b.capacity, b.point_list, b.ranges, b.tile_order = capacity, p(point_list), p(ranges), p(tile_order)
    ws = None
    if with_workspace:
        n = _lib.lib().fsgs_bin_workspace_bytes(W, H, capacity)
        ws = torch.empty(n, device=dev, dtype=torch.uint8)
        b.workspace, b.workspace_bytes = p(ws), n
    _lib.check(entry(ctypes.byref(b), ops._stream()), "binning")
    torch.cuda.synchronize()
    return ranges, point_list, tile_order


def test_noalloc_binning_equals_workspace_binning_twice_in_a_row():
    from fsgs import _lib, ops
    lib = _lib.lib()
    for P, W, H, ls, seed in ((40_000, 640, 480, -3.4, 21), (9_000, 200, 120, -2.2, 22)):
        s, cam = make_scene(P, W, H, seed=seed, log_scale_mean=ls)
        o = ops.preprocess_launch(W, H, 3, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"], s["sh_rest"],
                                  cam["Tw2v"], cam["Tv2s"], cam["campos"])
        n_slots, n_pairs = (int(v) for v in o["counters"][:2].tolist())
        assert 0 < n_pairs <= n_slots <= (1 << 20)
        ref_ranges, ref_list, ref_order = _bin(lib.fsgs_bin_tiles, W, H, o, s["opac"], n_slots, True)
        got_ranges, got_list, got_order = _bin(lib.fsgs_bin_tiles_noalloc, W, H, o, s["opac"], n_slots, False)
        assert torch.equal(got_ranges, ref_ranges)
        assert torch.equal(got_list, ref_list)
        assert sorted(got_order.tolist()) == list(range(ref_order.numel()))
        lens = (ref_ranges[:, 1] - ref_ranges[:, 0])
        assert bool((lens[got_order.long()][:-1] // 16 >= lens[got_order.long()][1:] // 16).all())
        assert int(o["counters"][2]) == 0  # nothing dropped


def test_noalloc_binning_allocates_nothing_and_works_at_its_limits():
    """What the entry point is for: with every input and output in place, a call changes neither the free device
    memory nor the framework's allocation count.  Checked on a frame close to both documented maxima (16 384 tiles,
    about 0.98 of the 2^20 pairs), compared element for element with the workspace path."""
    from fsgs import _lib, ops
    lib = _lib.lib()
    P, W, H = 100_000, 2048, 2048
    s, cam = make_scene(P, W, H, seed=23, log_scale_mean=-4.5)
    o = ops.preprocess_launch(W, H, 3, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"], s["sh_rest"],
                              cam["Tw2v"], cam["Tv2s"], cam["campos"])
    n_pairs = int(o["counters"][1])
    capacity = 1 << 20
    assert ((W + 15) // 16) * ((H + 15) // 16) == 16384 and 0.8 * capacity < n_pairs <= capacity
    ref_ranges, ref_list, _ = _bin(lib.fsgs_bin_tiles, W, H, o, s["opac"], capacity, True)
    _bin(lib.fsgs_bin_tiles_noalloc, W, H, o, s["opac"], capacity, False)      # the set-up call on this device
    # second call with every buffer made beforehand: nothing may be allocated while it runs
    dev = s["opac"].device
    T = 16384
    ranges = torch.full((T, 2), -7, device=dev, dtype=torch.int64)
    point_list = torch.full((capacity,), -7, device=dev, dtype=torch.int32)
    tile_order = torch.full((T,), -7, device=dev, dtype=torch.int32)
    b = _lib.BinArgs()
    b.P, b.W, b.H = P, W, H
    p = ops._ptr
    b.means2D, b.inverse_m, b.depths, b.opac = p(o["means2D"]), p(o["inverse_m"]), p(o["depths"]), p(s["opac"])
    b.radii, b.tile_counts, b.counters = p(o["radii"]), p(o["tile_counts"]), p(o["counters"])
    b.capacity, b.point_list, b.ranges, b.tile_order = capacity, p(point_list), p(ranges), p(tile_order)
    stream = ops._stream()
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    segments_before = torch.cuda.memory_stats()["segment.all.allocated"]
    _lib.check(lib.fsgs_bin_tiles_noalloc(ctypes.byref(b), stream), "binning")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == allocated_before
    assert torch.cuda.memory_stats()["segment.all.allocated"] == segments_before
    assert torch.equal(ranges, ref_ranges) and torch.equal(point_list, ref_list)
    assert int(o["counters"][2]) == 0


def test_noalloc_binning_rejects_sizes_beyond_its_fixed_scratch():
    from fsgs import _lib, ops
    lib = _lib.lib()
    dev = "cuda"
    one = torch.zeros(16, device=dev)
    b = _lib.BinArgs()
    b.P, b.W, b.H = 0, 64, 64
    cnt = torch.zeros(16, device=dev, dtype=torch.int32)
    ctr = torch.zeros(4, device=dev, dtype=torch.int64)
    out = torch.zeros(64, device=dev, dtype=torch.int64)
    p = ops._ptr
    b.tile_counts, b.counters, b.ranges, b.tile_order, b.point_list = p(cnt), p(ctr), p(out), p(cnt), p(one)
    b.capacity = (1 << 20) + 1
    assert lib.fsgs_bin_tiles_noalloc(ctypes.byref(b), ops._stream()) == -5  # FSGS_ERR_LIMIT: too many pairs
    b.capacity, b.W, b.H = 16, 16 * 200, 16 * 100
    assert lib.fsgs_bin_tiles_noalloc(ctypes.byref(b), ops._stream()) == -5  # 20 000 tiles > 16 384
    assert b"maximum" in lib.fsgs_status_string(-5)
    torch.cuda.synchronize()
