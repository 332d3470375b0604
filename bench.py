#!/usr/bin/env python
"""Benchmark of the surfel-rendering hot path: dynamic training step, 300k surfels @ 800x800.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload train_300k_800]

One step = LBS warp + preprocess + tile binning + compositing forward, compositing backward + preprocess
backward + LBS backward on a given upstream image gradient, fused visibility-masked Adam; with N > 1 every rank
renders its own view and the per-Gaussian gradients are all-reduced (NCCL) before Adam.  Prints ONE JSON line.

  value      view-iterations / s over all ranks, inputs resident in HBM, device-timed (CUDA events, max over ranks)
  e2e        the same step through fsgs.scene.DynamicScene.train_step with the step's inputs (camera, superpoint
             motion, upstream gradient) copied from pinned host memory and a scalar read back, every step; the
             upload of step i+1 runs on a copy stream beside step i and the scalar is read one step late
             (fsgs.feed.HostFeed / ScalarReader)
  roofline   the dominant kernel (compositing backward): algorithmic HBM bytes per launch / mean launch time
  cpu_baseline  the CPU oracle (a port of the reference's algorithm) on the host cores, same workload
  reference_cuda  the reference's own CUDA kernels (oracle/_ref, when built) on the same GPU, same step

--impl reference times the CPU oracle port alone (all host threads) and prints the same line shape.
"""
import argparse
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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_300k_800")
    ap.add_argument("--no-baselines", action="store_true", help="skip the CPU / reference-CUDA legs")
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


def build_workload(name, rank, device):
    """Scene parameters (identical on every rank), this rank's view and its upstream gradient, all on the CPU
    first (seeded), then moved."""
    from fsgs import workloads as wl
    cfg = wl.CONFIGS[name]
    P, W, H = cfg["P"], cfg["W"], cfg["H"]
    surf = wl.surfels(P, seed=0, log_scale_mean=cfg["log_scale_mean"], log_scale_std=cfg["log_scale_std"])
    M, K = cfg.get("M", 512), cfg.get("K", 3)
    sp = wl.superpoints(surf["means"], M=M, seed=rank)  # every view has its own time step -> its own motion
    centres = wl.superpoints(surf["means"], M=M, seed=0)["centres"]
    sp["centres"] = centres
    eye = (0.0, 0.0, 4.0) if rank == 0 else wl.sphere_eye(4.0, rank)
    cam = wl.camera(W, H, eye=eye)
    g = torch.Generator().manual_seed(100 + rank)
    g_img = torch.randn(3, H, W, generator=g)
    g_op = torch.randn(H, W, generator=g)
    return dict(cfg=cfg, P=P, W=W, H=H, M=M, K=K, surf=surf, sp=sp, centres=centres, cam=cam, g_img=g_img, g_op=g_op)


def cpu_step(wlk, steps):
    """The CPU oracle's version of one training step (warp by torch on the CPU, the rest in C); returns s/step."""
    import oracle as orc
    s, cam, W, H = wlk["surf"], wlk["cam"], wlk["W"], wlk["H"]
    P = wlk["P"]
    sp, c = wlk["sp"], wlk["centres"]
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
        gr = orc.render_backward(m2d, no, col, tm, im, None, fw[1], fw[2], wlk["g_img"], wlk["g_op"],
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


def reference_cuda_step(wlk, steps, warmup):
    """The same step on the reference's own CUDA kernels (oracle/_ref), called the way its Python does
    (debug=True in the preprocess; LBS warp and its adjoint by PyTorch ops).  Returns ms/step or None."""
    d = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(d):
        return None
    sys.path.insert(0, d)
    try:
        import _C as ref
    except ImportError:
        return None
    import oracle as orc
    from fsgs import ops
    dev = "cuda"
    s = {k: v.to(dev) for k, v in wlk["surf"].items()}
    cam = {k: v.to(dev) for k, v in wlk["cam"].items()}
    sp = {k: v.to(dev) for k, v in wlk["sp"].items()}
    c = wlk["centres"].to(dev)
    W, H, P = wlk["W"], wlk["H"], wlk["P"]
    d2, idx = ops.knn(s["means"], c, wlk["K"])
    w = torch.softmax(-d2, dim=-1)
    q = sp["sp_q"]
    t = sp["sp_t_raw"] + c - orc.quat_rotate(q, c)
    g_img, g_op, g_ext = wlk["g_img"].to(dev), wlk["g_op"].to(dev), torch.zeros(8, H, W, device=dev)
    g_sets, tick = [(g_img, g_op), (-g_img, -g_op)], [0]   # sign alternates as in run_ours
    leaves = [s[k].clone().requires_grad_() for k in ("means", "log_scales", "rots_raw", "opac_raw", "sh_dc", "sh_rest")]
    state = [(torch.zeros_like(p), torch.zeros_like(p)) for p in leaves]

    def step():
        g_img, g_op = g_sets[tick[0] & 1]
        tick[0] += 1
        xyz, ls, rr, orw, dc, rest = leaves
        means, scales, rots = orc.lbs_warp(xyz, ls, rr, idx, w, q, t, sp["sp_dr"], sp["sp_ds"])
        opac = torch.sigmoid(orw)
        m2d0 = torch.zeros(P, 2, device=dev)
        pre = ref.gs_2d_fast_preprocess_forward(W, H, 3, False, means.detach(), scales.detach(), rots.detach(),
                                                opac.detach(), dc.detach(), rest.detach(), cam["Tw2v"], cam["Tv2c"],
                                                cam["Tv2s"], cam["campos"], None, m2d0, None, True)
        m2d, col, tm, im, no, dep, rad, rng, pl = pre
        fw = ref.GS_2D_fast_render_forward(W, H, 0.2, 100.0, False, m2d, col, no, tm, im, pl, rng, None, None, None,
                                           None, None)
        gr = ref.GS_2D_fast_render_backward(m2d, no, col, tm, im, None, fw[0], fw[1], fw[2], None, g_img, g_op, g_ext,
                                            None, rng, pl, fw[4], 0.2, 100.0, None, None, None, None, None, None)
        gm, gs, gq, go = (torch.zeros_like(x) for x in (means, scales, rots, opac))
        gdc, grest = torch.zeros_like(dc), torch.zeros_like(rest)
        ref.gs_2d_fast_preprocess_backward(W, H, 3, False, means.detach(), scales.detach(), rots.detach(),
                                           opac.detach(), dc.detach(), rest.detach(), cam["Tw2v"], cam["Tv2s"],
                                           cam["campos"], tm, rad, col, no, gr[1], gr[2], gr[3], None, gr[0], gr[4],
                                           gm, gs, gq, go, gdc, grest, None, None)
        torch.autograd.backward([means, scales, rots, opac], [gm, gs, gq, go])
        dc.grad, rest.grad = gdc, grest
        vis = rad > 0
        for p, (m, v) in zip(leaves, state):
            ref.AdamMasksedUpdated(p.data, p.grad, m, v, vis, 1.6e-4, 0.9, 0.999, 1e-15, P, p.numel() // P)
            p.grad = None

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_ours(args):
    import torch.distributed as dist
    from fsgs import ops
    from fsgs.scene import DynamicScene, motion_at
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path in the product)"
    torch.cuda.set_device(local)
    distributed = world > 1
    if distributed:
        # the step's exchanges are 59 MB and 12 MB: at these sizes NCCL's ring all-reduce measured faster on the
        # 8-GPU NVSwitch box than its default choice (in-switch NVLS reduction), 0.216 + 0.077 ms against
        # 0.257 + 0.095 ms in isolation and 1.57 against 1.70 ms for the whole step; an explicit setting wins
        # (with two ranks NCCL's own choice was 2 % faster than the ring, so it is left alone there;
        # FSGS_BENCH_NCCL_ALGO=default|Ring|... overrides)
        algo = os.environ.get("FSGS_BENCH_NCCL_ALGO", "Ring" if world >= 4 else "default")
        if algo != "default":
            os.environ.setdefault("NCCL_ALGO", algo)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    wlk = build_workload(args.workload, rank, dev)
    W, H, P = wlk["W"], wlk["H"], wlk["P"]
    # every group at the position learning rate
    lr = 1.6e-4
    scene = DynamicScene(wlk["surf"], wlk["centres"], K=wlk["K"], device=dev,
                         lrs=dict(xyz=lr, sh_dc=lr, sh_rest=lr, opacity=lr, scaling=lr, rotation=lr))
    cam = {k: v.to(dev) for k, v in wlk["cam"].items()}
    motion = motion_at(wlk["sp"], wlk["centres"], dev)
    # The upstream gradient changes sign every step: Adam's first moment then oscillates about zero and the scene
    # stays where it is, so every phase of the run (and the reference arm) sees the same workload.  With a fixed
    # gradient Adam walks the scales and opacities steadily one way and the step gets cheaper as the run goes on.
    g_img, g_op = wlk["g_img"].to(dev), wlk["g_op"].to(dev)
    g_sets = [(g_img, g_op), (-g_img, -g_op)]
    tick = [0]

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    host_ms = {}

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        h0 = time.perf_counter()
        for _ in range(steps):
            fn()
        host_ms[fn.__name__] = (time.perf_counter() - h0) * 1e3 / steps  # time the host needs to queue one step
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if distributed:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    # ---- device-resident steps (value) ----
    def step():
        gi, go = g_sets[tick[0] & 1]
        tick[0] += 1
        scene.train_step(cam, (W, H), motion, gi, go, distributed=distributed)

    def fwd_only():
        with torch.no_grad():
            scene.render(cam, (W, H), motion)

    allreduce_ms = None
    if distributed:
        # communicator set-up: NCCL builds its channels lazily at the first collectives of each size class, which
        # would otherwise land in the first timed steps; these exchanges carry zeros and touch no training state.
        # The same buffers then time the two exchanges of a step in isolation (reported beside the step time).
        P = wlk["P"]
        allreduce_ms = []
        for n in (49 * P, 10 * P):
            z = torch.zeros(n, device=dev)
            for _ in range(5):
                dist.all_reduce(z)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                dist.all_reduce(z)
            e1.record()
            torch.cuda.synchronize()
            allreduce_ms.append(round(e0.elapsed_time(e1) / 10, 4))
            del z
    sampler = ClockSampler(local) if rank == 0 else None  # its child process starts while the warm-up runs
    for _ in range(max(args.warmup, 3)):
        step()
    scene.check()
    pairs_first = last_pairs(scene)
    if rank == 0:
        sampler.mark_start()
    ms_step = timed(step, args.steps)
    if rank == 0:
        sampler.mark_stop()
    clocks = sampler.stop() if rank == 0 else None
    scene.check()
    # the same K steps once more with every launch of this library bracketed by CUDA events (per-kernel times)
    ops.TIMERS = {}
    ms_step_instrumented = timed(step, args.steps)
    per_kernel = ops.timer_summary()
    ops.TIMERS = None
    ms_fwd = timed(fwd_only, args.steps)
    # ---- end to end: inputs from pinned host memory, a scalar back, every step ----
    hosts = [{"cam": {k: v.pin_memory() for k, v in wlk["cam"].items()},
              "motion": {k: v.cpu().pin_memory() for k, v in motion.items()},
              "g_img": (sgn * wlk["g_img"]).pin_memory(), "g_op": (sgn * wlk["g_op"]).pin_memory()}
             for sgn in (1.0, -1.0)]
    host = hosts[0]
    h2d = sum(v.numel() * 4 for v in host["cam"].values()) + sum(v.numel() * 4 for v in host["motion"].values()) + \
        host["g_img"].numel() * 4 + host["g_op"].numel() * 4
    sink = []
    from fsgs.feed import HostFeed, ScalarReader
    feed, reader = HostFeed(dev), ScalarReader(lag=1)
    feed.stage(hosts[tick[0] & 1])

    def e2e_step():
        tick[0] += 1
        feed.stage(hosts[tick[0] & 1])   # the next step's upload runs beside this step's kernels
        x = feed.take()
        out = scene.train_step(x["cam"], (W, H), x["motion"], x["g_img"], x["g_op"], distributed=distributed)
        feed.release()
        reader.push(out["opacity"].detach().mean())
        v = reader.pop()                 # device -> host read of the previous step's result, every step
        if v is not None:
            sink.append(float(v))

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    scene.check()

    pairs = list_pairs(scene)
    pairs_last = last_pairs(scene)

    # the same step with upstream gradients on the auxiliary channels too (normal and distortion losses switched on):
    # the compositing backward then carries 21 instead of 15 gradient components per splat
    gen = torch.Generator().manual_seed(300 + rank)
    g_nrm, g_dist = torch.randn(3, H, W, generator=gen).to(dev), (0.1 * torch.randn(1, H, W, generator=gen)).to(dev)
    g_aux = [{"normals": sgn * g_nrm, "distortion": sgn * g_dist} for sgn in (1.0, -1.0)]

    def step_aux():
        gi, go = g_sets[tick[0] & 1]
        ga = g_aux[tick[0] & 1]
        tick[0] += 1
        scene.train_step(cam, (W, H), motion, gi, go, distributed=distributed, g_aux=ga)

    for _ in range(3):
        step_aux()
    ms_step_aux = timed(step_aux, args.steps)
    pairs_aux = last_pairs(scene)

    # the step as a trainer runs it: target image in HBM, fused L1 + SSIM loss kernels produce the image gradient
    target = torch.rand(3, H, W, generator=torch.Generator().manual_seed(400 + rank)).to(dev)
    scene_l = DynamicScene(wlk["surf"], wlk["centres"], K=wlk["K"], device=dev,
                           lrs=dict(xyz=lr, sh_dc=lr, sh_rest=lr, opacity=lr, scaling=lr, rotation=lr))

    def step_loss():
        scene_l.train_step_with_loss(cam, (W, H), motion, target, distributed=distributed)

    for _ in range(3):
        step_loss()
    ops.TIMERS = {}
    ms_step_loss = timed(step_loss, args.steps)
    loss_kernels = ops.timer_summary()
    ops.TIMERS = None
    del scene_l

    line = None
    if rank == 0:
        peak, peak_kind = peaks()
        n_bwd, ms_bwd = per_kernel.get("blend_backward", (0, float("nan")))
        HW = W * H
        # compositing backward without auxiliary gradients, algorithmic bytes per launch: per list entry its id (4 B),
        # its 112-byte record and one reduction per gradient component (15 x 4 B); per pixel the upstream colour and
        # opacity gradients, the forward opacity and the last contributor (24 B)
        bwd_bytes = pairs * (4 + 112 + 4 * 15) + HW * 24
        achieved = bwd_bytes / (ms_bwd * 1e-3) / 1e9
        # algorithmic HBM bytes per launch of the bandwidth-bound stages (P Gaussians, V visible, 4-byte floats):
        #   adam: 58 floats x (param, grad, 2 moments read; param, 2 moments written) per visible Gaussian + the mask
        #   preprocess forward (LBS fused): 256 B of parameters in, 284 B of per-Gaussian outputs out (128 B record)
        #   preprocess backward: 376 B in (matrices, their gradients, SH), 240 B of parameter gradients out
        #   LBS backward: 96 B in, 48 B out per Gaussian, plus 56 B gathered per (Gaussian, neighbour) pair
        with torch.no_grad():
            V = int(scene.render(cam, (W, H), motion)["visibility_filter"].sum())
        stage_bytes = {"adam_masked_multi": V * 58 * 28 + P, "preprocess_forward": P * 540,
                       "preprocess_backward": P * 616, "lbs_warp_backward": P * (144 + 56 * wlk["K"])}
        hbm_stages = {}
        for k, b in stage_bytes.items():
            if k in per_kernel:
                gbs = b / (per_kernel[k][1] * 1e-3) / 1e9
                hbm_stages[k] = {"bytes": b, "GB/s": round(gbs, 1), "frac": round(gbs / peak, 3)}
        launches_per_step = sum(n for n, _ in per_kernel.values()) / args.steps + 4  # bin_tiles = 4 kernels, LBS adjoint = 2
        line = {
            "metric": METRIC, "value": world * 1e3 / ms_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "surfels": P, "image": [W, H], "superpoints": wlk["M"],
                       "knn": wlk["K"], "sh_degree": 3, "adam_lr": 1.6e-4, "views_per_step_per_gpu": 1,
                       "pairs_per_view": pairs, "pairs_first_last": [pairs_first, pairs_last],
                       "upstream_gradient": "fixed random image gradient, sign flipped every step",
                       "l2": "per-step working set (parameters, Adam state, gradients, records, images: > 400 MB) "
                             "exceeds the 126 MB L2; no explicit flush"},
            "fwd_frames_per_s": world * 1e3 / ms_fwd, "ms_per_fwd_frame": ms_fwd,
            "ms_per_step_with_aux_gradients": ms_step_aux, "pairs_after_aux_phase": pairs_aux,
            "ms_per_step_with_l1_ssim_loss": ms_step_loss,
            "loss_kernels_ms": {k: round(v[1], 4) for k, v in sorted(loss_kernels.items()) if k.startswith("ssim")},
            "e2e": {"value": world * 1e3 / ms_e2e, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4 + 32},
            "gpu_launches": int(round(launches_per_step * args.steps)),
            "kernels_ms": {k: round(v[1], 4) for k, v in sorted(per_kernel.items())},
            "ms_per_step_with_event_pairs": ms_step_instrumented,
            "roofline": {"kernel": "blend_backward", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
                         "algorithmic_bytes": bwd_bytes,
                         "note": "compositing is bound by instruction issue, not by HBM: the fraction is small by construction"},
            "hbm_stages": hbm_stages,
            "host_ms_per_step": {k: round(v, 4) for k, v in host_ms.items()},
            "allreduce_ms_49P_10P_floats": allreduce_ms,
            "clocks": clocks,
        }
        if world == 1 and not args.no_baselines:
            import oracle as orc
            n_cpu = 5
            sec = cpu_step(wlk, n_cpu)
            line["cpu_baseline"] = {"value": 1.0 / sec, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
                                    "sample": f"median of {n_cpu} full steps of the same workload"}
            ms_ref = reference_cuda_step(wlk, max(10, args.steps // 2), 3)
            if ms_ref is not None:
                line["reference_cuda"] = {"value": 1e3 / ms_ref, "unit": UNIT, "ms_per_step": ms_ref,
                                          "how": "reference kernels (oracle/_ref, sm_100, -O3) called as its Python "
                                                 "calls them (debug=True); LBS warp by PyTorch ops"}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def list_pairs(scene):
    from fsgs.renderer import list_capacity
    cap = list_capacity(scene.xyz.device)
    cap.poll(wait=True)
    return int(cap.high_water)


def last_pairs(scene):
    from fsgs.renderer import list_capacity
    cap = list_capacity(scene.xyz.device)
    cap.poll(wait=True)
    return int(cap.last_pairs)


def run_reference(args):
    """The reference arm: the CPU port of the reference's algorithm on the host cores, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import oracle as orc
    wlk = build_workload(args.workload, 0, "cpu")
    for _ in range(min(args.warmup, 1)):
        cpu_step(wlk, 1)
    n = max(1, min(args.steps, 8))
    t0 = time.perf_counter()
    sec = cpu_step(wlk, n)
    value = 1.0 / sec
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
            "warmup": min(args.warmup, 1), "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "surfels": wlk["P"], "image": [wlk["W"], wlk["H"]]},
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
