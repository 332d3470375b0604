#!/usr/bin/env python
"""Benchmark of the surfel-rendering hot path: dynamic training step, 300k surfels @ 800x800.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload train_300k_800]
                    [--views V | --batch-views B] [--repeats R] [--no-baselines]

One step = for every view of this rank: sigmoid + LBS warp + preprocess + tile binning + compositing forward,
compositing backward + preprocess backward + LBS backward on a given upstream image gradient (two C-ABI calls per
view, gradients of the views summed in place); with N > 1 ONE exchange of the summed per-Gaussian gradients and the
visibility mask (NCCL all-reduce); fused visibility-masked Adam.  Prints ONE JSON line.

  value      view-iterations / s over all ranks, inputs resident in HBM, device-timed (CUDA events, max over ranks),
             median over --repeats runs of --steps steps (min / max beside it)
  e2e        the same step with every view's inputs (camera, superpoint motion, upstream gradient) copied from pinned
             host memory and a scalar read back, every step; the upload of step i+1 runs on a copy stream beside step i
             and the scalar is read one step late (fsgs.feed.HostFeed / ScalarReader)
  roofline   the dominant kernel (compositing backward) against the FP32 pipe: 85 FLOP x contributing (pixel, entry)
             pairs, counted exactly by a replay kernel outside the timed region, / mean launch time; `stages` holds
             every stage's time with its own roofline (HBM for the per-Gaussian stages, FP32 for compositing)
  cpu_baseline    the CPU oracle (a port of the reference's algorithm) on the host cores, same workload, and what one
                  repetition of the reference's own PyTorch compositor costs on a stated crop
  reference_cuda  the reference's own CUDA kernels (oracle/_ref, when built) on the same GPU: the step as its Python
                  runs it, its forward alone, and every operator alone
  knn        exact k-NN of the two configurations that name one, beside torch.cdist + topk on the host cores

--impl reference times the reference's CPU path (the oracle port, all host threads) alone, same line shape.
--batch-views B: a fixed batch of B views sharded over the ranks (strong scaling) instead of --views per rank.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "fast-sp-gs_b200"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "train_iters_per_s"
UNIT = "iters/s"
STAGES = ["preprocess_forward", "bin_tiles", "blend_forward", "blend_backward", "preprocess_backward", "lbs_backward"]
# DRAM bytes (read + write) of one compositing-backward launch, from ncu captures of this command's workload
# (profiles/blend_kernels_*.md): workload -> bytes
NCU_TRAFFIC_BLEND_BACKWARD = {"train_300k_800": 53.728e6 + 1.317e6}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed runs of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_300k_800")
    ap.add_argument("--exchange", default="factors", choices=["factors", "rows"],
                    help="multi-GPU: all-gather the six SH-gradient factors per Gaussian and view (default) or "
                         "all-reduce the 48 SH gradient floats themselves")
    ap.add_argument("--views", type=int, default=1, help="views per rank per step (weak scaling)")
    ap.add_argument("--batch-views", type=int, default=0, help="views per step in total, sharded over the ranks")
    ap.add_argument("--no-baselines", action="store_true", help="skip the CPU / reference-CUDA / k-NN legs")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


_SAMPLER_CHILD = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
uuid, index = sys.argv[1], int(sys.argv[2])
try:
    h = nv.nvmlDeviceGetHandleByUUID(uuid) if uuid else nv.nvmlDeviceGetHandleByIndex(index)
except Exception:
    h = nv.nvmlDeviceGetHandleByIndex(index)
try:
    print("max", nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
except Exception:
    print("max", -1, flush=True)
while True:
    try:
        mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        try:
            bits = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
        except AttributeError:
            bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        print(repr(time.time()), mhz, bits, flush=True)
    except Exception:
        pass
    time.sleep(0.002)
"""


class ClockSampler:
    """SM clock and clock-event (throttle) reasons sampled through NVML while the timed region runs: read-only
    queries every 2 ms from a child process (a thread of this process competes with the launching thread for the
    interpreter lock and may get a single sample in a 40 ms region).  The child is started before the warm-up;
    ``mark_start`` / ``mark_stop`` bracket the timed region and only the samples between them are reported."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index):
        self.proc, self.lines, self.t0, self.t1 = None, [], None, None
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(gpu_index).uuid)
        except Exception:
            uuid = ""
        try:
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_CHILD, uuid, str(gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError as e:
            self.error = f"sampler not started: {e}"

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.split())

    def mark_start(self):
        deadline = time.time() + 5.0  # the child needs a moment to import and initialise NVML
        while self.proc is not None and len(self.lines) < 2 and time.time() < deadline:
            time.sleep(0.005)
        self.t0 = time.time()

    def mark_stop(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error], "samples": 0}
        time.sleep(0.01)
        self.proc.terminate()
        self.thread.join(timeout=2)
        mx = next((int(l[1]) for l in self.lines if l and l[0] == "max"), None)
        rows = [(float(l[0]), int(l[1]), int(l[2])) for l in self.lines if len(l) == 3 and l[0] != "max"]
        inside = [r for r in rows if self.t0 is not None and self.t0 <= r[0] <= self.t1]
        sm = sorted(r[1] for r in inside)
        bits = 0
        for r in inside:
            bits |= r[2]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": mx if mx and mx > 0 else None,
                "reasons": sorted(n for b, n in self.REASONS.items() if bits & b), "samples": len(sm)}


class LaunchTimer:
    """Brackets every call of one C-ABI entry point with a pair of CUDA events on torch's current stream, by
    swapping the attribute of the loaded library handle for the duration of a ``with`` block (bench only)."""

    def __init__(self, name):
        from fsgs._lib import lib
        self.handle, self.name, self.events = lib(), name, []

    def __enter__(self):
        self.orig = getattr(self.handle, self.name)

        def wrapped(*a):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = self.orig(*a)
            e1.record()
            self.events.append((e0, e1))
            return rc
        setattr(self.handle, self.name, wrapped)
        return self

    def __exit__(self, *exc):
        setattr(self.handle, self.name, self.orig)

    def total_ms(self):
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.events), len(self.events)


def stage_times():
    """(ms, launches) per stage recorded by the library since ``fsgs_stage_timing(1)`` (synchronises)."""
    from fsgs._lib import check, lib
    ms, n = (ctypes.c_float * len(STAGES))(), (ctypes.c_int32 * len(STAGES))()
    check(lib().fsgs_stage_times(ms, n), "fsgs_stage_times")
    return {k: (float(ms[i]), int(n[i])) for i, k in enumerate(STAGES)}


# ---------------------------------------------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------------------------------------------

def view_inputs(cfg, surf, view_id):
    """Camera, superpoint motion draw and upstream gradient of global view number ``view_id`` (CPU tensors, seeded by
    the view number alone, so every rank and every arm derives the same view)."""
    from fsgs import workloads as wl
    W, H = cfg["W"], cfg["H"]
    if "views" in cfg:
        eye = wl.arc_eye(cfg["radius"], view_id % cfg["views"], cfg["views"])
    else:
        eye = (0.0, 0.0, 4.0) if view_id == 0 else wl.sphere_eye(4.0, view_id)
    g = torch.Generator().manual_seed(100 + view_id)
    return dict(cam=wl.camera(W, H, eye=eye), sp=wl.superpoints(surf["means"], M=cfg.get("M", 512), seed=view_id),
                g_img=torch.randn(3, H, W, generator=g), g_op=torch.randn(H, W, generator=g))


def build_workload(name, view_ids):
    """Scene parameters (identical on every rank) and this rank's views, all on the CPU (seeded)."""
    from fsgs import workloads as wl
    cfg = wl.CONFIGS[name]
    surf = wl.surfels(cfg["P"], seed=0, log_scale_mean=cfg["log_scale_mean"], log_scale_std=cfg["log_scale_std"])
    M, K = cfg.get("M", 512), cfg.get("K", 3)
    centres = wl.superpoints(surf["means"], M=M, seed=0)["centres"]
    views = [view_inputs(cfg, surf, v) for v in view_ids]
    return dict(cfg=cfg, P=cfg["P"], W=cfg["W"], H=cfg["H"], M=M, K=K, surf=surf, centres=centres, views=views)


# ---------------------------------------------------------------------------------------------------------------
# baselines
# ---------------------------------------------------------------------------------------------------------------

def cpu_step(wlk, steps):
    """The CPU oracle's version of one training step on the first view (warp by torch on the CPU, the rest in C);
    returns the median s/step."""
    import oracle as orc
    s, W, H, P = wlk["surf"], wlk["W"], wlk["H"], wlk["P"]
    v = wlk["views"][0]
    cam, sp, c = v["cam"], v["sp"], wlk["centres"]
    d2, idx = orc.knn(s["means"], c, wlk["K"])
    w = torch.softmax(-d2, dim=-1)
    q = sp["sp_q"]
    t = sp["sp_t_raw"] + c - orc.quat_rotate(q, c)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        with torch.no_grad():
            means, scales, rots = orc.lbs_warp(s["means"], s["log_scales"], s["rots_raw"], idx, w, q, t, sp["sp_dr"],
                                               sp["sp_ds"])
        pre = orc.preprocess_forward(W, H, 3, means, scales, rots, s["opac"], s["sh_dc"], s["sh_rest"], cam["Tw2v"],
                                     cam["Tv2s"], cam["campos"])
        m2d, col, tm, im, no, dep, rad, rng, pl = pre[:9]
        fw = orc.render_forward(W, H, 0.2, 100.0, False, m2d, col, no, tm, im, pl, rng)
        gr = orc.render_backward(m2d, no, col, tm, im, None, fw[1], fw[2], v["g_img"], v["g_op"],
                                 torch.zeros(8, H, W), None, rng, pl, fw[4], 0.2, 100.0)
        pg = orc.preprocess_backward(W, H, 3, means, scales, rots, s["sh_dc"], s["sh_rest"], cam["Tw2v"], cam["Tv2s"],
                                     cam["campos"], tm, rad, col, gr[1], gr[2], gr[3], gr[0], gr[4])
        vis = rad > 0
        for prm, g_ in ((s["means"], pg[0]), (s["log_scales"], pg[1]), (s["rots_raw"], pg[2]), (s["opac_raw"], pg[3]),
                        (s["sh_dc"], pg[4]), (s["sh_rest"], pg[5])):
            prm = prm.clone()
            orc.adam(prm, g_, torch.zeros_like(prm), torch.zeros_like(prm), vis, 1e-3, 0.9, 0.999, 1e-15, P,
                     prm.numel() // P)
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2]


_PY_COMPOSITOR_CHILD = r"""
import json, os, sys, time
ROOT, crop, P = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
sys.path[:0] = [os.path.join(ROOT, "fast-sp-gs_b200"), os.path.join(ROOT, "oracle")]
import torch
torch.set_num_threads(os.cpu_count())
import refpy
refpy.import_reference(native=None)
from fast_2d_gs.renderer import gs_2d_fast_render as R
import oracle as orc
from fsgs import workloads as wl
W = H = 800
s = wl.surfels(P, seed=0, log_scale_mean=-4.5)
cam = wl.camera(W, H)
# a crop x crop window at the image centre: same camera, principal point shifted
Tv2s = cam["Tv2s"].clone()
Tv2s[0, 2] -= (W - crop) / 2
Tv2s[1, 2] -= (H - crop) / 2
pre = orc.preprocess_forward(crop, crop, 3, s["means"], s["scales"], s["rots"], s["opac"], s["sh_dc"], s["sh_rest"],
                             cam["Tw2v"], Tv2s, cam["campos"])
m2d, col, tm, im, no, dep, rad, rng, pl = pre[:9]
n_real = int(pre[10])
pl = pl[:n_real].contiguous()
ins = [t.clone().requires_grad_() for t in (m2d, col, no, tm)]
t0 = time.perf_counter()
img, opa, ext, nc = R.GS_2D_fast_rasterize(crop, crop, ins[0], ins[1], ins[2], ins[3], im, rng, pl.long(), 0.2, 100.,
                                           False)
t1 = time.perf_counter()
g = torch.Generator().manual_seed(1)
torch.autograd.backward([img, opa], [torch.randn(img.shape, generator=g), torch.randn(opa.shape, generator=g)])
t2 = time.perf_counter()
# the same crop through the C port, for the ratio
t3 = time.perf_counter()
fw = orc.render_forward(crop, crop, 0.2, 100.0, False, m2d, col, no, tm, im, pre[8], rng)
t4 = time.perf_counter()
print(json.dumps({"pairs": n_real, "fwd_s": t1 - t0, "bwd_s": t2 - t1, "port_fwd_s": t4 - t3,
                  "threads": torch.get_num_threads(), "max_abs_vs_port": float((img.detach() - fw[0]).abs().max())}))
"""


def reference_pytorch_compositor(P, crop=128, timeout=600):
    """One repetition of the reference's own PyTorch compositor (``GS_2D_fast_rasterize``,
    renderer/gs_2d_fast_render.py:433-555, forward and autograd backward) on the host cores, on a centre crop of the
    800x800 frame of the workload (the whole frame takes minutes); in a child process.  None when the reference's
    Python is not available."""
    if not os.path.isdir(os.path.join(ROOT, "oracle", "_ref", "py", "fast_2d_gs")):
        return None
    try:
        r = subprocess.run([sys.executable, "-c", _PY_COMPOSITOR_CHILD, ROOT, str(crop), str(P)], capture_output=True,
                           text=True, timeout=timeout)
        if r.returncode != 0:
            return {"error": r.stderr.strip().splitlines()[-1][:200] if r.stderr.strip() else "failed"}
        d = json.loads(r.stdout.strip().splitlines()[-1])
    except (subprocess.TimeoutExpired, ValueError) as e:
        return {"error": str(e)[:200]}
    d["sample"] = f"{crop}x{crop} centre crop of the 800x800 frame, {P} surfels, 1 repetition, forward + autograd backward"
    d["port_speedup_fwd"] = d["fwd_s"] / max(d["port_fwd_s"], 1e-9)
    return d


def _ref_module():
    d = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(d):
        return None
    if d not in sys.path:
        sys.path.insert(0, d)
    try:
        import _C as ref
        return ref
    except ImportError:
        return None


def _event_ms(fn, n, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def reference_cuda(wlk, steps, warmup):
    """The reference's own CUDA kernels (oracle/_ref) on the first view: (a) the training step called the way its
    Python does (debug=True in the preprocess, as ``_Fast_Render`` passes it; LBS warp and its adjoint by PyTorch
    ops); (b) its forward alone (frames/s); (c) every operator alone with debug=False.  None when not built."""
    ref = _ref_module()
    if ref is None:
        return None
    import oracle as orc
    from fsgs import ops
    dev = "cuda"
    v = wlk["views"][0]
    s = {k: t.to(dev) for k, t in wlk["surf"].items()}
    cam = {k: t.to(dev) for k, t in v["cam"].items()}
    sp = {k: t.to(dev) for k, t in v["sp"].items()}
    c = wlk["centres"].to(dev)
    W, H, P = wlk["W"], wlk["H"], wlk["P"]
    d2, idx = ops.knn(s["means"], c, wlk["K"])
    w = torch.softmax(-d2, dim=-1)
    q = sp["sp_q"]
    t = sp["sp_t_raw"] + c - orc.quat_rotate(q, c)
    g_img, g_op, g_ext = v["g_img"].to(dev), v["g_op"].to(dev), torch.zeros(8, H, W, device=dev)
    g_sets, tick = [(g_img, g_op), (-g_img, -g_op)], [0]   # sign alternates as in run_ours
    leaves = [s[k].clone().requires_grad_() for k in ("means", "log_scales", "rots_raw", "opac_raw", "sh_dc", "sh_rest")]
    state = [(torch.zeros_like(p), torch.zeros_like(p)) for p in leaves]
    keep = {}

    def forward(debug=True):
        xyz, ls, rr, orw, dc, rest = leaves
        means, scales, rots = orc.lbs_warp(xyz, ls, rr, idx, w, q, t, sp["sp_dr"], sp["sp_ds"])
        opac = torch.sigmoid(orw)
        m2d0 = torch.zeros(P, 2, device=dev)
        pre = ref.gs_2d_fast_preprocess_forward(W, H, 3, False, means.detach(), scales.detach(), rots.detach(),
                                                opac.detach(), dc.detach(), rest.detach(), cam["Tw2v"], cam["Tv2c"],
                                                cam["Tv2s"], cam["campos"], None, m2d0, None, debug)
        m2d, col, tm, im, no, dep, rad, rng, pl = pre
        fw = ref.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, m2d, col, no, tm, im, pl, rng, None, None, None,
                                           None, None)
        keep.update(means=means, scales=scales, rots=rots, opac=opac, pre=pre, fw=fw)

    def step():
        gi, go = g_sets[tick[0] & 1]
        tick[0] += 1
        xyz, ls, rr, orw, dc, rest = leaves
        forward(True)
        means, scales, rots, opac, pre, fw = (keep[k] for k in ("means", "scales", "rots", "opac", "pre", "fw"))
        m2d, col, tm, im, no, dep, rad, rng, pl = pre
        gr = ref.GS_2D_fast_render_backward(m2d, no, col, tm, im, None, fw[0], fw[1], fw[2], None, gi, go, g_ext,
                                            None, rng, pl, fw[4], 0.2, 100.0, None, None, None, None, None, None)
        gm, gs, gq, gop = (torch.zeros_like(x) for x in (means, scales, rots, opac))
        gdc, grest = torch.zeros_like(dc), torch.zeros_like(rest)
        ref.gs_2d_fast_preprocess_backward(W, H, 3, False, means.detach(), scales.detach(), rots.detach(),
                                           opac.detach(), dc.detach(), rest.detach(), cam["Tw2v"], cam["Tv2s"],
                                           cam["campos"], tm, rad, col, no, gr[1], gr[2], gr[3], None, gr[0], gr[4],
                                           gm, gs, gq, gop, gdc, grest, None, None)
        keep.update(gr=gr)
        torch.autograd.backward([means, scales, rots, opac], [gm, gs, gq, gop])
        dc.grad, rest.grad = gdc, grest
        vis = rad > 0
        for p, (m, vv) in zip(leaves, state):
            ref.AdamMasksedUpdated(p.data, p.grad, m, vv, vis, 1.6e-4, 0.9, 0.999, 1e-15, P, p.numel() // P)
            p.grad = None

    # its Python synchronises with the device several times per step (debug=True reads counters back), so a step's
    # time follows the host's mood: median of three runs, all three reported
    step_runs = sorted(_event_ms(step, steps, warmup if r == 0 else 0) for r in range(3))
    ms_step = step_runs[1]
    with torch.no_grad():
        ms_fwd = sorted(_event_ms(lambda: forward(True), steps, 2 if r == 0 else 0) for r in range(3))[1]
    # every operator alone, debug=False, on the tensors of the last step
    means, scales, rots, opac, pre, fw, gr = (keep[k].detach() if torch.is_tensor(keep[k]) else keep[k]
                                              for k in ("means", "scales", "rots", "opac", "pre", "fw", "gr"))
    m2d, col, tm, im, no, dep, rad, rng, pl = pre
    dc, rest = leaves[4].detach(), leaves[5].detach()
    gbuf = [torch.zeros_like(x) for x in (means, scales, rots, opac, dc, rest)]
    ops_ms = {
        "preprocess_forward_with_binning": _event_ms(lambda: ref.gs_2d_fast_preprocess_forward(
            W, H, 3, False, means, scales, rots, opac, dc, rest, cam["Tw2v"], cam["Tv2c"], cam["Tv2s"], cam["campos"],
            None, torch.zeros(P, 2, device=dev), None, False), steps),
        "blend_forward": _event_ms(lambda: ref.GS_2D_fast_render_forward(
            W, H, 0.2, 100.0, False, m2d, col, no, tm, im, pl, rng, None, None, None, None, None), steps),
        "blend_backward": _event_ms(lambda: ref.GS_2D_fast_render_backward(
            m2d, no, col, tm, im, None, fw[0], fw[1], fw[2], None, g_img, g_op, g_ext, None, rng, pl, fw[4], 0.2,
            100.0, None, None, None, None, None, None), steps),
        "preprocess_backward": _event_ms(lambda: ref.gs_2d_fast_preprocess_backward(
            W, H, 3, False, means, scales, rots, opac, dc, rest, cam["Tw2v"], cam["Tv2s"], cam["campos"], tm, rad, col,
            no, gr[1].clone(), gr[2], gr[3], None, gr[0], gr[4], *gbuf, None, None), steps),
        "adam_six_launches": _event_ms(lambda: [ref.AdamMasksedUpdated(
            p.data, torch.zeros_like(p), m, vv, rad > 0, 1.6e-4, 0.9, 0.999, 1e-15, P, p.numel() // P)
            for p, (m, vv) in zip(leaves, state)], steps),
    }
    return {"value": 1e3 / ms_step, "unit": UNIT, "ms_per_step": ms_step,
            "ms_per_step_runs": [round(x, 4) for x in step_runs], "fwd_frames_per_s": 1e3 / ms_fwd,
            "ms_per_fwd_frame": ms_fwd, "operators_alone_ms": {k: round(x, 4) for k, x in ops_ms.items()},
            "operators_alone_sum_ms": round(sum(ops_ms.values()), 4),
            "how": "reference kernels (oracle/_ref, sm_100, -O3). value / fwd: called as its Python calls them "
                   "(debug=True as _Fast_Render passes it; sigmoid, LBS warp and their adjoints by PyTorch ops). "
                   "operators_alone_ms: each operator by itself with debug=False, CUDA events around the call "
                   "(its own allocations, zero fills and the device-to-host read of the pair count included)"}


def knn_legs(no_cpu=False):
    """Exact k-NN of the two configurations that name one: 100k x 512 (k = 3) and 2 M x 4096 (k = 8), device-timed;
    beside them torch.cdist + topk on the host cores (the reference's form, network.py:787-788), bounded in size."""
    from fsgs import ops, workloads as wl
    out = {}
    for tag, N, M, K in (("c1_100k_x_512_k3", 100_000, 512, 3), ("c5_2m_x_4096_k8", 2_000_000, 4096, 8)):
        x, c = wl.knn_points_c1(N, M, seed=0)
        xd, cd = x.cuda(), c.cuda()
        ms = _event_ms(lambda: ops.knn(xd, cd, K, method="brute"), 10, 3)
        ms_grid = _event_ms(lambda: ops.knn(xd, cd, K, method="grid"), 10, 3)
        flop = 8.0 * N * M
        e = {"ms_brute_force": round(ms, 4), "gflop_8NM": flop / 1e9, "tflops_brute_force": flop / (ms * 1e-3) / 1e12,
             "ms_grid": round(ms_grid, 4), "note": "grid: same distances and indices bit for bit, fewer evaluations"}
        if not no_cpu:
            n_cpu = min(N, 200_000)
            torch.set_num_threads(os.cpu_count())
            t0 = time.perf_counter()
            d = torch.cdist(x[:n_cpu], c)
            d.topk(K, dim=-1, largest=False)
            sec = time.perf_counter() - t0
            e["torch_cpu"] = {"ms_scaled_to_N": sec * 1e3 * N / n_cpu, "rows_timed": n_cpu,
                              "threads": torch.get_num_threads()}
        out[tag] = e
        del xd, cd
    return out


# ---------------------------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------------------------

def run_ours(args):
    import torch.distributed as dist
    from fsgs._lib import check, lib
    from fsgs.dist import shard_views
    from fsgs.feed import HostFeed, ScalarReader
    from fsgs.scene import DynamicScene, motion_at
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path in the product)"
    torch.cuda.set_device(local)
    distributed = world > 1
    if distributed:
        # the step's exchanges are 59 MB and 12 MB: at these sizes NCCL's ring all-reduce measured faster on the
        # 8-GPU NVSwitch box than its default choice (in-switch NVLS reduction); an explicit NCCL_ALGO wins, and
        # FSGS_BENCH_NCCL_ALGO=default|Ring|... overrides (with two ranks NCCL's own choice was 2 % faster)
        algo = os.environ.get("FSGS_BENCH_NCCL_ALGO", "Ring" if world >= 4 else "default")
        if algo != "default":
            os.environ.setdefault("NCCL_ALGO", algo)
        # NCCL's kernels on a high-priority stream: the step's collectives are meant to run under the adjoint and
        # optimiser kernels, whose grids fill every SM; at equal priority a collective's blocks (which each want most
        # of an SM) were not placed until those grids had drained, and the exchange ran after them instead of beside
        # them (FSGS_BENCH_NCCL_PRIORITY=0 restores torch's default)
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = os.environ.get("FSGS_BENCH_NCCL_PRIORITY", "1") != "0"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=opts)
    dev = torch.device("cuda", local)
    if args.batch_views > 0:
        view_ids, scaling, total_views = shard_views(args.batch_views, rank, world), "strong", args.batch_views
    else:
        view_ids = [rank * args.views + j for j in range(args.views)]
        scaling, total_views = "weak", world * args.views
    wlk = build_workload(args.workload, view_ids)
    W, H, P, K, M = wlk["W"], wlk["H"], wlk["P"], wlk["K"], wlk["M"]
    # view slots per rank in the exchange (the same number on every rank) and the form of the exchange
    xch = dict(views_per_rank=max(1, -(-total_views // world)), exchange=args.exchange)
    knn_every_step = args.workload.startswith("stress")  # that configuration recomputes the k-NN every step
    lr = 1.6e-4  # every group at the position learning rate
    new_scene = lambda: DynamicScene(wlk["surf"], wlk["centres"], K=K, device=dev,
                                     lrs=dict(xyz=lr, sh_dc=lr, sh_rest=lr, opacity=lr, scaling=lr, rotation=lr))
    scene = new_scene()
    # The upstream gradient changes sign every step: Adam's first moment then oscillates about zero and the scene
    # stays where it is, so every phase of the run (and the reference arm) sees the same workload.  With a fixed
    # gradient Adam walks the scales and opacities steadily one way and the step gets cheaper as the run goes on.
    dev_views = []
    for v in wlk["views"]:
        cam = {k: t.to(dev) for k, t in v["cam"].items()}
        motion = motion_at(v["sp"], wlk["centres"], dev)
        gi, go = v["g_img"].to(dev), v["g_op"].to(dev)
        dev_views.append([dict(cam=cam, motion=motion, g_images=s * gi, g_opacity=s * go) for s in (1.0, -1.0)])
    tick = [0]

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    host_ms = {}

    def timed(fn, steps, label=None, repeats=1):
        """Median (and all) device ms/step over ``repeats`` runs of ``steps`` calls, max over ranks per run."""
        runs = []
        for _ in range(repeats):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            h0 = time.perf_counter()
            for _ in range(steps):
                fn()
            host = (time.perf_counter() - h0) * 1e3 / steps  # time the host needs to queue one step
            e1.record()
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if distributed:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            runs.append(float(ms) / steps)
            if label:
                host_ms.setdefault(label, []).append(host)
        runs.sort()
        return runs[len(runs) // 2], runs

    def step():
        k = tick[0] & 1
        tick[0] += 1
        if knn_every_step:
            scene.refresh_knn()
        scene.train_views([v[k] for v in dev_views], (W, H), distributed=distributed, **xch)

    def fwd_only():
        eng = scene._engine((W, H))
        for v in dev_views:
            eng.forward(scene, v[0]["cam"], v[0]["motion"])

    allreduce_ms, exchange_ms = None, {}
    if distributed:
        # communicator set-up: NCCL builds its channels lazily at the first collectives of each size class, which
        # would otherwise land in the first timed steps; these exchanges carry zeros and touch no training state.
        # The same buffers then time the two exchanges of a step in isolation (reported beside the step time).
        allreduce_ms = []
        for n in (49 * P, 10 * P):
            z = torch.zeros(n, device=dev)
            for _ in range(5):
                dist.all_reduce(z)
            torch.cuda.synchronize()
            dist.barrier()
            allreduce_ms.append(round(_event_ms(lambda: dist.all_reduce(z), 10, 0), 4))
            del z
        # the factor exchange's all-gather (7 floats per Gaussian and view slot); a P-float all-reduce for scale
        zs = torch.zeros(xch["views_per_rank"] * 7 * P, device=dev)
        zr = torch.zeros(world * zs.numel(), device=dev)
        zm = torch.zeros(P, device=dev)
        for _ in range(5):
            dist.all_gather_into_tensor(zr, zs)
            dist.all_reduce(zm)
        torch.cuda.synchronize()
        dist.barrier()
        exchange_ms["all_gather_7P_per_slot"] = round(_event_ms(lambda: dist.all_gather_into_tensor(zr, zs), 10, 0), 4)
        exchange_ms["all_reduce_P"] = round(_event_ms(lambda: dist.all_reduce(zm), 10, 0), 4)
        del zs, zr, zm
    sampler = ClockSampler(local) if rank == 0 else None  # its child process starts while the warm-up runs
    for _ in range(max(args.warmup, 3)):
        step()
    scene.check()
    pairs_first = scene.engine.last_pairs
    if rank == 0:
        sampler.mark_start()
    ms_step, step_runs = timed(step, args.steps, "step", max(1, args.repeats))
    if rank == 0:
        sampler.mark_stop()
    clocks = sampler.stop() if rank == 0 else None
    scene.check()
    n_views = len(dev_views)

    # the same K steps once more with every stage bracketed by CUDA events inside the library (per-stage times)
    check(lib().fsgs_stage_timing(1), "fsgs_stage_timing")
    with LaunchTimer("fsgs_adam_masked_multi_fmask") as adam_t:
        ms_step_staged, _ = timed(step, args.steps, "step_with_stage_events")
    per_stage = stage_times()
    check(lib().fsgs_stage_timing(0), "fsgs_stage_timing")
    adam_ms, adam_calls = adam_t.total_ms()
    ms_fwd, fwd_runs = timed(fwd_only, args.steps, "forward", max(1, args.repeats))
    scene.check()

    # work of one view, counted exactly by the replay kernel (first local view)
    counts = torch.zeros(3, dtype=torch.int64, device=dev)
    vis_count = pairs = 0
    if n_views:
        eng = scene._engine((W, H))
        eng.forward(scene, dev_views[0][0]["cam"], dev_views[0][0]["motion"])
        check(lib().fsgs_view_pair_counts(ctypes.byref(eng._args), ctypes.c_void_p(counts.data_ptr()),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "pair counts")
        vis_count = int((eng.radii > 0).sum())
        eng.check()
        pairs = eng.last_pairs
    traversed, contributing, bwd_walked = (int(x) for x in counts.tolist())

    # ---- end to end: every view's inputs from pinned host memory, a scalar back, every step ----
    hosts = []
    for sgn in (1.0, -1.0):
        hosts.append({f"v{j}": {"cam": {k: t.pin_memory() for k, t in v["cam"].items()},
                                "motion": {k: t.cpu().pin_memory() for k, t in dev_views[j][0]["motion"].items()},
                                "g_img": (sgn * v["g_img"]).pin_memory(), "g_op": (sgn * v["g_op"]).pin_memory()}
                      for j, v in enumerate(wlk["views"])})
    nbytes = lambda d: sum(nbytes(x) if isinstance(x, dict) else x.numel() * x.element_size() for x in d.values())
    h2d = nbytes(hosts[0])
    sink = []
    feed, reader = HostFeed(dev), ScalarReader(lag=1)
    if n_views:
        feed.stage(hosts[tick[0] & 1])

    def e2e_step():
        tick[0] += 1
        if knn_every_step:
            scene.refresh_knn()
        if not n_views:
            scene.train_views([], (W, H), distributed=distributed, **xch)
            return
        feed.stage(hosts[tick[0] & 1])   # the next step's upload runs beside this step's kernels
        x = feed.take()
        views = [dict(cam=x[f"v{j}"]["cam"], motion=x[f"v{j}"]["motion"], g_images=x[f"v{j}"]["g_img"],
                      g_opacity=x[f"v{j}"]["g_op"]) for j in range(n_views)]
        eng = scene.train_views(views, (W, H), distributed=distributed, **xch)
        feed.release()
        reader.push(eng.opacity.mean())
        val = reader.pop()               # device -> host read of the previous step's result, every step
        if val is not None:
            sink.append(float(val))

    for _ in range(3):
        e2e_step()
    ms_e2e, e2e_runs = timed(e2e_step, args.steps, "e2e_step", max(1, args.repeats))
    scene.check()
    pairs_last = scene.engine.last_pairs

    # the same step with upstream gradients on the auxiliary channels too (normal and distortion losses switched on):
    # the compositing backward then carries 21 instead of 15 gradient components per splat
    ms_step_aux = ms_step_loss = None
    if n_views:
        gen = torch.Generator().manual_seed(300 + rank)
        g_ext = torch.zeros(8, H, W)
        g_ext[1:4] = torch.randn(3, H, W, generator=gen)
        g_ext[5] = 0.1 * torch.randn(H, W, generator=gen)
        g_ext = g_ext.to(dev)
        aux_views = [[dict(v[k], g_extras=(1.0, -1.0)[k] * g_ext) for k in (0, 1)] for v in dev_views]

        def step_aux():
            k = tick[0] & 1
            tick[0] += 1
            scene.train_views([v[k] for v in aux_views], (W, H), distributed=distributed, **xch)

        for _ in range(3):
            step_aux()
        ms_step_aux, _ = timed(step_aux, args.steps, "step_aux")
        # the step as a trainer runs it: target image in HBM, fused L1 + SSIM loss kernels produce the image gradient
        target = torch.rand(3, H, W, generator=torch.Generator().manual_seed(400 + rank)).to(dev)
        scene_l = new_scene()
        v0 = dev_views[0][0]

        def step_loss():
            scene_l.train_step_with_loss(v0["cam"], (W, H), v0["motion"], target, distributed=distributed)

        for _ in range(3):
            step_loss()
        ms_step_loss, _ = timed(step_loss, args.steps, "step_loss")
        del scene_l

    # the step with the superpoint motion produced by the deformation network at a time t (network trained as well,
    # kernel-weighted LBS weights re-evaluated and trained): what the reference's iteration does before its render
    ms_step_motion = motion_ms = motion_pairs = None
    if n_views:
        from fsgs.motion import MotionNet
        net = MotionNet(M, device=dev, local_frame=True, seed=1)
        # The network's learning rate is 1e-6 here, not the trainer's 1.6e-4: the upstream gradient is noise whose sign
        # alternates, and while that keeps the Gaussians in place (each parameter moves by +-lr), a step of 1.6e-4 on
        # all 523 k weights at once moves the network's OUTPUT by a tenth of the scene and the scene then drifts
        # (pair count x 30 within 30 steps).  Every kernel of the step runs the same at either rate;
        # `motion_net_pairs_first_last` in the output shows that the workload stayed put.
        scene_m = DynamicScene(wlk["surf"], wlk["centres"], K=K, device=dev, motion_net=net,
                               kernel_weights=(torch.full((M,), -1.5), torch.zeros(M)), lr_deform=1e-6,
                               lrs=dict(xyz=lr, sh_dc=lr, sh_rest=lr, opacity=lr, scaling=lr, rotation=lr))
        t_views = [[dict(cam=v[k]["cam"], t=torch.tensor([0.1 + 0.8 * j / max(n_views, 1)], device=dev),
                         g_images=v[k]["g_images"], g_opacity=v[k]["g_opacity"]) for k in (0, 1)]
                   for j, v in enumerate(dev_views)]

        def step_motion():
            k = tick[0] & 1
            tick[0] += 1
            scene_m.train_views([v[k] for v in t_views], (W, H), distributed=distributed, **xch)

        for _ in range(3):
            step_motion()
        scene_m.check()
        motion_pairs = [scene_m.engine.last_pairs]
        ms_step_motion, _ = timed(step_motion, args.steps, "step_motion_net")
        scene_m.check()
        motion_pairs.append(scene_m.engine.last_pairs)
        t0 = t_views[0][0]["t"]
        gp = torch.zeros_like(net.params.data)
        gm = {k: torch.randn_like(x) for k, x in net.forward(scene_m.centres, t0).items()}
        motion_ms = {"forward": round(_event_ms(lambda: net.forward(scene_m.centres, t0, out=scene_m.motion_buf), 50, 5), 4),
                     "backward": round(_event_ms(lambda: net.backward(gm, gp), 50, 5), 4),
                     "net": f"{net.cfg.depth} x {net.cfg.width}, {M} superpoints, {net.params.numel()} parameters"}
        del scene_m

    # ---- where the time of a multi-rank step goes: CUDA events at the phase boundaries of train_views, one step at a
    # time (synchronised, so the absolute times sit a little above the pipelined step), rank 0, outside timed regions
    timeline = None
    if distributed and n_views:
        acc, n_trace = {}, 20
        for it in range(n_trace):
            scene.trace = []
            step()
            torch.cuda.synchronize()
            t0 = scene.trace[0][1]
            for label, ev in scene.trace[1:]:
                acc[label] = acc.get(label, 0.0) + t0.elapsed_time(ev)
        scene.trace = None
        timeline = {k: round(v / n_trace, 4) for k, v in acc.items()}

    # ---- replicas must stay identical; a split batch must equal the serial one (outside every timed region) ----
    checks = None
    if distributed:
        worst = torch.zeros(1, device=dev)
        for p in scene.params:
            ref_p = p.detach().clone()
            dist.broadcast(ref_p, 0)
            worst = torch.maximum(worst, (p.detach() - ref_p).abs().max().reshape(1))
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        # views 0, 1, 2 of the batch dealt to the ranks as shard_views deals them (with two ranks: two views and one,
        # so a view slot stays empty; with more than three ranks some ranks have none) against all three on every
        # rank, serially
        cfg, surf = wlk["cfg"], wlk["surf"]
        two = []
        for vid in (0, 1, 2):
            v = view_inputs(cfg, surf, vid)
            two.append(dict(cam={k: t.to(dev) for k, t in v["cam"].items()}, motion=motion_at(v["sp"], wlk["centres"], dev),
                            g_images=v["g_img"].to(dev), g_opacity=v["g_op"].to(dev)))
        mine = [two[v] for v in shard_views(3, rank, world)]
        slots = -(-3 // world)
        a, b = new_scene(), new_scene()
        # The summed gradients of the first step (same parameters on both sides: only the summation differs), then
        # the parameters after a second step.  Adam's first steps are lr * g / |g|: a gradient within summation noise
        # of zero moves its parameter by +-lr either way, the second step's gradients then see different parameters,
        # and the parameter comparison sits a decade or two above the gradient comparison.
        # The yardstick: the serial step run twice.  The compositing adjoint sums each Gaussian's per-tile
        # contributions with floating-point atomics, whose order differs from run to run; through the cancelling
        # terms of the splat-matrix adjoint that leaves about 1e-5 on the scale and rotation gradients (1e-7 on the
        # others) between two runs of the very same step.
        rel, rel_g, rel_noise = (torch.zeros(1, device=dev) for _ in range(3))
        c = new_scene()
        for it in range(2):
            a.train_views(mine, (W, H), distributed=True, views_per_rank=slots, exchange=args.exchange)
            b.train_views(two, (W, H), distributed=False)
            if it == 0:
                c.train_views(two, (W, H), distributed=False)
                per_tensor = torch.zeros(6, 2, device=dev)   # position, SH DC, SH rest, opacity, scale, rotation
                for k, (x, y, z) in enumerate(zip(a.params, b.params, c.params)):
                    gx, gy, gz = a.bucket.view_of(x), b.bucket.view_of(y), c.bucket.view_of(z)
                    per_tensor[k, 0] = (gx - gy).norm() / gy.norm().clamp_min(1e-30)
                    per_tensor[k, 1] = (gz - gy).norm() / gy.norm().clamp_min(1e-30)
                rel_g, rel_noise = per_tensor[:, 0].max().reshape(1), per_tensor[:, 1].max().reshape(1)
        del c
        dist.all_reduce(per_tensor, op=dist.ReduceOp.MAX)
        for x, y in zip(a.params, b.params):
            rel = torch.maximum(rel, ((x.detach() - y.detach()).norm() / y.detach().norm().clamp_min(1e-30)).reshape(1))
        dist.all_reduce(rel, op=dist.ReduceOp.MAX)
        dist.all_reduce(rel_g, op=dist.ReduceOp.MAX)
        dist.all_reduce(rel_noise, op=dist.ReduceOp.MAX)
        checks = {"replica_max_abs_diff_after_run": float(worst),
                  "three_views_dealt_to_the_ranks_vs_serial_rel_l2": float(rel),
                  "three_views_dealt_to_the_ranks_vs_serial_first_step_gradients_rel_l2": float(rel_g),
                  "serial_step_run_twice_first_step_gradients_rel_l2": float(rel_noise),
                  "first_step_gradients_rel_l2_per_tensor": {
                      name: {"dealt_vs_serial": float(per_tensor[k, 0]), "serial_vs_serial": float(per_tensor[k, 1])}
                      for k, name in enumerate(("xyz", "sh_dc", "sh_rest", "opacity", "scaling", "rotation"))}}
        del a, b

    if rank == 0:
        peak, peak_kind = peaks()
        clock_mhz = (clocks or {}).get("sm_mhz") or (clocks or {}).get("sm_max_mhz") or 1965
        fp32_peak = 148 * 128 * 2 * clock_mhz * 1e6 / 1e12  # TFLOP/s
        HW = W * H
        V, R = vis_count, pairs
        per_launch = {k: (ms / n if n else None) for k, (ms, n) in per_stage.items()}
        per_launch["adam_masked_multi"] = adam_ms / max(adam_calls // 2, 1) if adam_calls else None  # 2 launches / step
        # algorithmic work per launch.  HBM stages: bytes by the per-unit figures of the reference's data layout --
        #   preprocess forward: 232 B of parameters per Gaussian in, 120 B per visible Gaussian out, 12 B per
        #     (Gaussian, neighbour) for the fused LBS warp; this library's own traffic (128-byte record besides the
        #     reference-layout outputs, warped parameters) is 540 B per Gaussian, given beside it
        #   binning: 100 B per visible Gaussian + 8 B key per pair out, then 8 B in + 4 B out per pair for the sort
        #   preprocess backward: 450 B in + 232 B out per visible Gaussian (own: 616 B per Gaussian, every row written)
        #   LBS backward: 144 B per Gaussian + 56 B gathered per (Gaussian, neighbour)
        #   Adam: 58 floats x (param, grad, 2 moments in; param, 2 moments out) per visible Gaussian + the mask
        # FP32 stages: compositing forward 65 FLOP per traversed pair (auxiliary channels on), backward 85 FLOP per
        # contributing pair (150 with auxiliary gradients)
        hbm_alg = {"preprocess_forward": 232 * P + 120 * V + 12 * K * P, "bin_tiles": 100 * V + 20 * R,
                   "preprocess_backward": 682 * V, "lbs_backward": P * (144 + 56 * K),
                   "adam_masked_multi": V * 58 * 28 + 4 * P}
        hbm_own = {"preprocess_forward": 540 * P, "preprocess_backward": 616 * P}
        flop_alg = {"blend_forward": 65.0 * traversed, "blend_backward": 85.0 * contributing}
        stages = {}
        for k, ms in per_launch.items():
            if ms is None:
                continue
            e = {"ms": round(ms, 4)}
            if k in hbm_alg:
                gbs = hbm_alg[k] / (ms * 1e-3) / 1e9
                e.update(bound="hbm", algorithmic_bytes=hbm_alg[k], achieved_GBs=round(gbs, 1), frac=round(gbs / peak, 3))
                if k in hbm_own:
                    e["frac_on_own_traffic"] = round(hbm_own[k] / (ms * 1e-3) / 1e9 / peak, 3)
            if k in flop_alg:
                tf = flop_alg[k] / (ms * 1e-3) / 1e12
                e.update(bound="fp32", algorithmic_flop=flop_alg[k], achieved_TFLOPs=round(tf, 2),
                         frac=round(tf / fp32_peak, 3))
            stages[k] = e
        ms_bwd = per_launch.get("blend_backward") or float("nan")
        achieved = flop_alg["blend_backward"] / (ms_bwd * 1e-3) / 1e12
        bwd_bytes = R * (4 + 112 + 4 * 15) + HW * 24
        traffic = NCU_TRAFFIC_BLEND_BACKWARD.get(args.workload)
        launches_per_step = n_views * 10 + 2  # per view: preprocess, 4 binning, compositing fwd; bwd, preprocess bwd, 2 LBS
        med = lambda xs: sorted(xs)[len(xs) // 2]
        line = {
            "metric": METRIC, "value": total_views * 1e3 / ms_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "repeats": {"n": len(step_runs), "ms_per_step_min": step_runs[0], "ms_per_step_max": step_runs[-1]},
            "config": {"workload": args.workload, "surfels": P, "image": [W, H], "superpoints": M, "knn": K,
                       "sh_degree": 3, "adam_lr": lr, "views_per_step": total_views,
                       "views_per_step_on_rank0": n_views, "knn_recomputed_every_step": knn_every_step,
                       "exchange": args.exchange if world > 1 else None,
                       "visible_on_view0": V, "pairs_on_view0": R, "pairs_first_last": [pairs_first, pairs_last],
                       "upstream_gradient": "fixed random image gradient per view, sign flipped every step",
                       "l2": "per-step working set (parameters, Adam state, gradients, records, images: > 400 MB) "
                             "exceeds the 126 MB L2; no explicit flush"},
            "fwd_frames_per_s": total_views * 1e3 / ms_fwd, "ms_per_fwd_batch": ms_fwd,
            "fwd_repeats": {"min": fwd_runs[0], "max": fwd_runs[-1]},
            "ms_per_step_with_aux_gradients": ms_step_aux, "ms_per_step_with_l1_ssim_loss": ms_step_loss,
            "ms_per_step_with_motion_net": ms_step_motion, "motion_net_pairs_first_last": motion_pairs,
            "motion_net_ms": motion_ms,
            "e2e": {"value": total_views * 1e3 / ms_e2e, "unit": UNIT, "ms_per_step": ms_e2e,
                    "ms_per_step_min_max": [e2e_runs[0], e2e_runs[-1]], "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4 + 32 * n_views},
            "gpu_launches": int(launches_per_step * args.steps),
            "gpu_launches_per_step": launches_per_step,
            "ms_per_step_with_stage_events": ms_step_staged,
            "roofline": {"kernel": "blend_backward", "bound": "fp32", "achieved": achieved, "peak": fp32_peak,
                         "unit": "TFLOP/s", "frac": achieved / fp32_peak,
                         "peak_kind": f"148 SM x 128 lanes x 2 x {clock_mhz} MHz (median SM clock sampled in the timed region)",
                         "algorithmic_flop": flop_alg["blend_backward"], "flop_per_contributing_pair": 85,
                         "contributing_pairs": contributing, "traversed_pairs": traversed,
                         "pairs_walked_by_backward": bwd_walked, "traffic": traffic,
                         "hbm": {"algorithmic_bytes": bwd_bytes, "achieved_GBs": bwd_bytes / (ms_bwd * 1e-3) / 1e9,
                                 "frac_of_hbm_peak": bwd_bytes / (ms_bwd * 1e-3) / 1e9 / peak, "peak_GBs": peak,
                                 "peak_kind": peak_kind}},
            "stages": stages,
            "host_ms_per_step": {k: round(med(v), 4) for k, v in host_ms.items()},
            "allreduce_ms_49P_10P_floats": allreduce_ms, "factor_exchange_ms": exchange_ms or None,
            "multi_gpu_checks": checks, "step_timeline_ms_rank0": timeline,
            "clocks": clocks,
        }
        if world == 1 and not args.no_baselines:
            import oracle as orc
            n_cpu = 5
            sec = cpu_step(wlk, n_cpu)
            line["cpu_baseline"] = {"value": 1.0 / sec, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                                    "sample": f"median of {n_cpu} full steps of the same workload (first view)",
                                    "reference_pytorch_compositor": reference_pytorch_compositor(P)}
            line["reference_cuda"] = reference_cuda(wlk, max(10, args.steps // 2), 3)
            line["knn"] = knn_legs()
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference arm: the reference's CPU path for this step (the oracle port, all host threads), rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count())  # a launcher may have set 1 for its ranks
    import oracle as orc
    orc.set_num_threads(os.cpu_count())
    torch.set_num_threads(os.cpu_count())
    wlk = build_workload(args.workload, [0])
    cfg = wlk["cfg"]
    warm = max(0, min(args.warmup, 2))
    for _ in range(warm):
        cpu_step(wlk, 1)
    n = max(1, min(args.steps, 8))   # bounded: one step is about a second of all cores
    t0 = time.perf_counter()
    sec = cpu_step(wlk, n)
    value = 1.0 / sec
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
            "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "surfels": wlk["P"], "image": [wlk["W"], wlk["H"]],
                       "superpoints": wlk["M"], "knn": wlk["K"], "sh_degree": 3, "adam_lr": 1.6e-4,
                       "views_per_step": 1, "steps_requested": args.steps, "warmup_requested": args.warmup,
                       "note": "one view on the host cores whatever --gpus says; steps capped at 8"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                             "sample": f"median of {n} full steps; wall {time.perf_counter() - t0:.1f} s"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
