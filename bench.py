#!/usr/bin/env python
"""Benchmark of the rasterizer hot path: fwd+bwd Mpix/s on synthetic aerial-city workloads.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

One "step" = one data-parallel training step of the hot path over a batch of cameras: for every camera
preprocess_gaussians -> (Gaussian all-to-all when N > 1) -> render_gaussians -> backward of both, through
the drop-in `diff_gaussian_rasterization` API.  Default workload: 6M Gaussians, 8 cameras 1600x1200
(the configuration the headline metric is quoted on); total work is fixed as N grows ("strong" scaling).

Prints ONE JSON line (rank 0).  `value` = whole-job Mpix/s with inputs resident in HBM; `e2e` = the same
step with the step's host inputs copied from pinned memory and its result read back inside the timed region.
`--impl reference` times the CPU oracle (the reference has no CPU implementation of its own; its rasterizer is
CUDA-only) on the host cores for a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "citygs-x_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402


# ----------------------------------------------------------------------------- workloads
WORKLOADS = {
    # name: (cfg id, description)
    "cfg0": (0, "50k Gaussians, 2 cameras 256x144 (CPU plumbing configuration: its CPU arm runs 2 gloo ranks)"),
    "cfg1": (1, "1M Gaussians, 1 camera 1920x1080 (single-GPU rasterizer fwd+bwd)"),
    "cfg2": (2, "6M Gaussians, 8 cameras 1600x1200 on a ring (data-parallel step)"),
    "cfg3": (3, "20M clustered Gaussians, 16 cameras 3840x2160 (load-imbalance stress)"),
    "cfg4": (4, "cfg2's scene at --gaussians N (capacity sweep), densification statistics updated every step"),
    "redistribute": (None, "anchor redistribution: --gaussians rows per job (default 6M) of model state (parameters + "
                           "both Adam moments + level tags, 916 bytes per row) moved to rank i % N in one exchange"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--gaussians", type=int, default=None, help="override the Gaussian count (scaling sweep)")
    ap.add_argument("--cameras", type=int, default=None, help="use only the first N cameras (profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-reference", action="store_true",
                    help="--impl reference: time the CPU oracle port even when the reference's CUDA extension is usable")
    ap.add_argument("--no-ref-gpu", action="store_true",
                    help="do not time the reference's CUDA extension beside this repository's arm (N=1)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="N>1: skip the correctness run on the reduced scene")
    ap.add_argument("--no-stage-events", action="store_true", help="do not bracket library calls with CUDA events")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample nvidia-smi during the run")
    ap.add_argument("--render-streams", type=int, default=None,
                    help="single-GPU step: cameras alternate between this many CUDA streams")
    ap.add_argument("--sort-variant", type=int, default=None,
                    help="A/B timing: select a sort variant through the library's test-only switch")
    ap.add_argument("--render-variant", type=int, default=None,
                    help="A/B timing: select a blending kernel variant through the library's test-only switch")
    ap.add_argument("--cpu-sample-gaussians", type=int, default=None)
    ap.add_argument("--kernel-table", action="store_true",
                    help="after the measurement, profile 3 more steps with torch.profiler on every rank and print "
                         "rank 0's per-kernel device times to stderr (for multi-GPU runs, where ncu is not used)")
    ap.add_argument("--densification-stats", action="store_true",
                    help="update the densification statistics inside every step (always on for cfg4)")
    return ap.parse_args()


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- reference / CPU arm
def workload_config(a, cams, n_scene):
    """The `config` object of the JSON line: the same for both arms of one workload."""
    return {"workload": a.workload, "description": WORKLOADS[a.workload][1], "gaussians": n_scene,
            "cameras": len(cams), "resolution": f"{cams[0].W}x{cams[0].H}",
            "l2": ("inputs larger than L2 (per-step working set of several GB)" if n_scene * len(cams) >= 4_000_000
                   else "per-step working set below the 126 MB L2, no flush between steps: warm-cache numbers"),
            "parallelism": f"gaussian-shard x tile-row split, ws={a.gpus}"}


_CPU_SCENES = {}


def cpu_step_sample(cfg, n_gauss, cam_idx=0):
    """One camera of the workload through the CPU oracle (fwd+bwd). Returns (seconds, Mpix, sample text).
    The scene is generated once per process, outside the timed part."""
    from cgx import synthetic as S
    from oracle import cpu_raster as O

    key = (cfg, n_gauss, cam_idx)
    if key not in _CPU_SCENES:
        g, cams = S.config(cfg, n_gaussians=n_gauss)
        cam = cams[cam_idx]
        g["rgb"] = S.colours_for(g, cam)
        g["all_map"] = S.build_all_map(g["means3D"], g["scales"], g["rotations"], cam)
        gen = torch.Generator().manual_seed(99)
        cot = dict(color=torch.randn(3, cam.H, cam.W, generator=gen),
                   all_map=torch.randn(5, cam.H, cam.W, generator=gen),
                   plane_depth=torch.randn(1, cam.H, cam.W, generator=gen))
        cd = dict(W=cam.W, H=cam.H, tanfovx=cam.tanfovx, tanfovy=cam.tanfovy, viewmatrix=cam.viewmatrix,
                  projmatrix=cam.projmatrix, bg=torch.zeros(3))
        O.lib()
        _CPU_SCENES[key] = (g, cam, cd, cot)
    g, cam, cd, cot = _CPU_SCENES[key]
    t0 = time.perf_counter()
    O.full_step(g, cd, cot=cot)
    dt = time.perf_counter() - t0
    P = g["means3D"].shape[0]
    return dt, cam.W * cam.H / 1e6, f"camera {cam_idx} of {P} Gaussians at {cam.W}x{cam.H}, fwd+bwd, oracle (C, OpenMP)"


def _cfg0_gloo_worker(rank, ws, port, steps, warmup, out_q):
    """One rank of the CPU plumbing configuration: oracle preprocess of the local shard for both cameras, the
    repository's own exchange over gloo (collective transport, CPU packing backend), oracle blending fwd+bwd of the
    local tile rows, reverse exchange, oracle preprocess backward."""
    import torch.distributed as dist
    from types import SimpleNamespace

    from cgx import exchange, synthetic as S
    from cgx import workload_division as WD
    from oracle import cpu_raster as O
    from oracle.exchange_backend import OracleBackend

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // ws))
    os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 2) // ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    g, cams = S.config(0)
    sel = slice(rank, None, ws)
    loc = {k: v[sel].contiguous() for k, v in g.items()}
    rgbs = [S.colours_for(loc, cam) for cam in cams]
    gen = torch.Generator().manual_seed(99)
    cots = [dict(color=torch.randn(3, c.H, c.W, generator=gen), all_map=torch.randn(5, c.H, c.W, generator=gen),
                 plane_depth=torch.randn(1, c.H, c.W, generator=gen)) for c in cams]
    ctx = WD.DivisionContext(image_height=cams[0].H, image_width=cams[0].W, rank=rank, world_size=ws, bsz=len(cams),
                             device="cpu")
    hist = WD.DivisionStrategyHistoryFinal(cams, ws, rank, ctx=ctx)
    rasts = [SimpleNamespace(raster_settings=SimpleNamespace(image_height=c.H, image_width=c.W)) for c in cams]
    args = [{"avoid_pixel_all2all": False} for _ in cams]
    be = OracleBackend()
    times = []
    for it in range(warmup + steps):
        dist.barrier()
        t0 = time.perf_counter()
        strategies, _ = WD.start_strategy_final(cams, hist, ctx=ctx)
        screen, pre = [], []
        for cam, rgb in zip(cams, rgbs):
            m2, dep, rad, cov3, co = O.preprocess_fwd(loc["means3D"], loc["scales"], loc["rotations"], loc["opacities"],
                                                      cam.viewmatrix, cam.projmatrix, cam.W, cam.H, cam.tanfovx,
                                                      cam.tanfovy)
            m2.requires_grad_(True)
            co.requires_grad_(True)
            pre.append((m2, co, rad, cov3))
            screen.append((m2, rgb, co, rad, dep, loc["means3D"], loc["scales"], loc["rotations"]))
        out = exchange.all_to_all_communication_final(rasts, screen, args, strategies, backend=be)
        m2r, rgbr, cor, radr, depr, m3r, scr, rotr = out[:8]
        heads, grads = [], []
        for k, cam in enumerate(cams):
            local = strategies[k].get_compute_locally()
            if local is None or m2r[k].shape[0] == 0:
                continue
            am = S.build_all_map(m3r[k], scr[k], rotr[k], cam)
            b = O.bin_and_sort(m2r[k].detach(), depr[k], radr[k], local, cam.W, cam.H)
            bg = torch.zeros(3)
            f = O.render_fwd(m2r[k].detach(), cor[k].detach(), rgbr[k], am, b["ranges"], b["point_list"], local, bg,
                             cam.W, cam.H, cam.tanfovx, cam.tanfovy)
            rb = O.render_bwd(m2r[k].detach(), cor[k].detach(), rgbr[k], am, f["out_all_map"], f["final_T"],
                              f["n_contrib_px"], b["ranges"], b["point_list"], local, bg, cam.W, cam.H, cam.tanfovx,
                              cam.tanfovy, cots[k]["color"], cots[k]["all_map"], cots[k]["plane_depth"])
            heads += [m2r[k], cor[k]]
            grads += [rb["dL_dmeans2D"], rb["dL_dconic_opacity"]]
        if not heads:
            heads, grads = [m2r[0].sum() * 0.0], [torch.zeros(())]
        torch.autograd.backward(heads, grads)           # the reverse exchange
        for (m2, co, rad, cov3), cam in zip(pre, cams):
            O.preprocess_bwd(loc["means3D"], loc["scales"], loc["rotations"], rad, cov3, cam.viewmatrix,
                             cam.projmatrix, cam.W, cam.H, cam.tanfovx, cam.tanfovy,
                             m2.grad if m2.grad is not None else torch.zeros_like(m2),
                             co.grad if co.grad is not None else torch.zeros_like(co))
            m2.grad = co.grad = None
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64)
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        if it >= warmup:
            times.append(float(dt))
    if rank == 0:
        out_q.put(times)
    dist.barrier()
    dist.destroy_process_group()


def cfg0_cpu_gloo(steps, warmup, ws=2):
    """Times the CPU plumbing configuration (50k Gaussians, two 256x144 cameras) on `ws` gloo ranks of this host.
    Returns (seconds per step: max over ranks, mean over steps; Mpix per step; sample text)."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cfg0_gloo_worker, args=(r, ws, port, steps, warmup, q)) for r in range(ws)]
    for p in procs:
        p.start()
    import queue

    times = None
    while times is None:
        try:
            times = q.get(timeout=2)
        except queue.Empty:
            if any(p.exitcode not in (None, 0) for p in procs):
                for p in procs:
                    p.kill()
                raise RuntimeError("a rank of the two-rank CPU configuration failed")
    for p in procs:
        p.join(timeout=60)
    return statistics.mean(times), 2 * 256 * 144 / 1e6, \
        f"full cfg0 step on {ws} gloo ranks (oracle kernels, this repository's exchange with all_to_all_single)"


class ReferenceCudaStep:
    """The same training step through the reference's OWN CUDA extension (oracle/_ref/cityx_ref_C.so, compiled from
    the reference's sources, unmodified), driven through its raw entry points in the order its Python package
    drives them: per camera preprocess_gaussians -> render_gaussians, then render_gaussians_backward ->
    preprocess_gaussians_backward, parameter gradients summed over the cameras.  Same scene, cameras, colours and
    upstream gradients as this repository's arm.  The per-Gaussian plane descriptors (`all_map`), which the
    reference's caller builds with a dozen tensor ops per camera per step, are computed ONCE outside the timed
    region and get no gradient here: that favours the reference."""

    LABELS = {"preprocess": ("10 preprocess",), "binning": ("24 updateDistributedStatLocally.updateTileTouched",
                                                             "30 InclusiveSum", "40 duplicateWithKeys"),
              "sort": ("50 SortPairs",), "tile_ranges": ("60 identifyTileRanges",), "render_fwd": ("70 render",),
              "render_bwd": ("b10 render",), "preprocess_bwd": ("b20 preprocess",)}

    def __init__(self, ref, g, cams, dev, seed=4242):
        from cgx import synthetic as S

        self.ref, self.cams, self.dev = ref, cams, dev
        names = ("means3D", "scales", "rotations", "opacities")
        self.host = {k: g[k].contiguous().pin_memory() for k in names}
        self.params = {k: v.to(dev) for k, v in self.host.items()}
        self.grad_host = {k: torch.empty_like(v).pin_memory() for k, v in self.host.items()}
        self.sh_dummy = torch.empty(0, device=dev)
        gd = {"means3D": self.params["means3D"], "sh": g["sh"].to(dev)}
        gen = torch.Generator().manual_seed(seed)
        self.view, self.proj, self.campos, self.rgb, self.all_map, self.cot_host, self.cot, self.local = \
            [], [], [], [], [], [], [], []
        for cam in cams:
            self.view.append(cam.viewmatrix.to(dev))
            self.proj.append(cam.projmatrix.to(dev))
            self.campos.append(cam.campos.to(dev))
            with torch.no_grad():
                self.rgb.append(S.colours_for(gd, cam))
                self.all_map.append(S.build_all_map(self.params["means3D"], self.params["scales"],
                                                    self.params["rotations"], cam))
            ch = [torch.randn(3, cam.H, cam.W, generator=gen), torch.randn(5, cam.H, cam.W, generator=gen),
                  torch.randn(1, cam.H, cam.W, generator=gen)]
            self.cot_host.append([c.pin_memory() for c in ch])
            self.cot.append([c.to(dev) for c in ch])
            self.local.append(torch.ones((cam.H + 15) // 16, (cam.W + 15) // 16, dtype=torch.bool, device=dev))
        del gd
        self.bg = torch.zeros(3, device=dev)
        self.h2d_bytes = sum(v.numel() * 4 for v in self.host.values()) + \
            sum(c.numel() * 4 for cs in self.cot_host for c in cs)
        self.d2h_bytes = sum(v.numel() * 4 for v in self.grad_host.values())
        self.grads = None
        self.iteration = 0

    def _args(self, timed_log=None):
        a = {"mode": "train", "world_size": "1", "global_rank": "0", "local_rank": "0", "mp_world_size": "1",
             "mp_rank": "0", "log_folder": timed_log or "/tmp", "log_interval": "2", "iteration": "2",
             "zhx_debug": "False", "zhx_time": "False", "dist_global_strategy": "", "avoid_pixel_all2all": False,
             "stats_collector": {}}
        if timed_log:            # the reference writes its own per-stage GPU timers when iteration % log_interval == 1
            a.update(zhx_time="True", iteration="1")
        return a

    def run(self, timed_log=None):
        ref, p = self.ref, self.params
        self.iteration += 1
        args = self._args(timed_log)
        saved = []
        for k, cam in enumerate(self.cams):
            _, means2D, depths, radii, cov3D, conic_opacity, rgb0, clamped = ref.preprocess_gaussians(
                p["means3D"], p["scales"], p["rotations"], self.sh_dummy, p["opacities"], 1.0, self.view[k],
                self.proj[k], cam.tanfovx, cam.tanfovy, cam.H, cam.W, 3, self.campos[k], False, False, args)
            (R, color, n_render, n_consider, n_contrib, observe, out_all_map, plane_depth, geomB, binB, imgB) = \
                ref.render_gaussians(self.bg, cam.H, cam.W, means2D, depths, radii, conic_opacity, self.rgb[k],
                                     self.local[k], self.view[k], self.campos[k], cam.tanfovx, cam.tanfovy,
                                     self.all_map[k], True, False, args)
            saved.append((means2D, radii, cov3D, conic_opacity, clamped, R, out_all_map, geomB, binB, imgB))
        total = None
        for k in reversed(range(len(self.cams))):
            cam = self.cams[k]
            means2D, radii, cov3D, conic_opacity, clamped, R, out_all_map, geomB, binB, imgB = saved.pop()
            d_m2, d_abs, d_co, d_rgb, d_map = ref.render_gaussians_backward(
                self.bg, cam.tanfovx, cam.tanfovy, out_all_map, self.all_map[k], R, geomB, binB, imgB, self.local[k],
                self.cot[k][0], self.cot[k][1], self.cot[k][2], means2D, conic_opacity, self.rgb[k], True, False, args)
            d_means, d_scales, d_rot, d_sh, d_op = ref.preprocess_gaussians_backward(
                radii, cov3D, clamped, p["means3D"], p["scales"], p["rotations"], self.sh_dummy, 1.0, self.view[k],
                self.proj[k], cam.tanfovx, cam.tanfovy, cam.H, cam.W, 3, self.campos[k], d_m2, d_co, d_rgb, R, False,
                args)
            if total is None:
                total = [d_means, d_scales, d_rot, d_op]
            else:
                for t, d in zip(total, (d_means, d_scales, d_rot, d_op)):
                    t += d
        self.grads = dict(zip(("means3D", "scales", "rotations", "opacities"), total))

    def run_e2e(self):
        for k, v in self.host.items():
            self.params[k].copy_(v, non_blocking=True)
        for dsts, srcs in zip(self.cot, self.cot_host):
            for d, s_ in zip(dsts, srcs):
                d.copy_(s_, non_blocking=True)
        self.run()
        for k, v in self.grads.items():
            self.grad_host[k].copy_(v, non_blocking=True)
        torch.cuda.synchronize()

    def stage_times(self):
        """One extra step with the reference's own per-stage GPU timers switched on (they write a log file)."""
        import re
        import tempfile

        out = {}
        with tempfile.TemporaryDirectory() as d:
            self.run(timed_log=d)
            torch.cuda.synchronize()
            text = "".join(p.read_text() for p in Path(d).glob("gpu_time_*.log"))
        found = {}
        for label, ms in re.findall(r"^(.+?) time: ([0-9.eE+-]+) ms$", text, flags=re.M):
            found.setdefault(label.strip(), []).append(float(ms))
        # every entry point owns its timer object and prints it once: each label appears once per camera
        for stage, labels in self.LABELS.items():
            out[stage] = sum(sum(found.get(lab, [])) for lab in labels)
        return out


def time_steps(fn, steps):
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def load_reference_extension():
    """The reference's CUDA extension when it has been built (oracle/build_ref.py) and a GPU is present."""
    if not torch.cuda.is_available():
        return None
    try:
        from oracle import build_ref

        return build_ref.load()
    except Exception as e:       # a broken checker must not take the bench down
        print(f"[bench] reference extension not usable: {e}", file=sys.stderr)
        return None


def measure_reference_gpu(a, g, cams, dev, steps, warmup, e2e=True, stages=True):
    ref = load_reference_extension()
    if ref is None:
        return None
    step = ReferenceCudaStep(ref, g, cams, dev)
    for _ in range(max(warmup, 1)):
        step.run()
    ms = time_steps(step.run, steps)
    out = {"ms_per_step": ms, "steps": steps}
    if e2e:
        step.run_e2e()
        out["e2e_ms_per_step"] = time_steps(step.run_e2e, steps)
        out["h2d_bytes_per_step"], out["d2h_bytes_per_step"] = step.h2d_bytes, step.d2h_bytes
    if stages:
        out["stages"] = step.stage_times()
    del step
    torch.cuda.empty_cache()
    return out


def run_reference_arm(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from cgx import synthetic as S

    cfg = WORKLOADS[a.workload][0]
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    torch.set_num_threads(cores)
    g, cams = S.config(cfg, n_gaussians=a.gaussians)
    if a.cameras:
        cams = cams[: a.cameras]
    n_scene = g["means3D"].shape[0]
    mpix_all = sum(c.W * c.H for c in cams) / 1e6
    line = {"impl": "reference", "metric": "fwd+bwd Mpix/s", "unit": "Mpix/s", "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(a, cams, n_scene)}
    gpu = None
    if a.workload != "cfg0" and not a.cpu_reference:
        if torch.cuda.is_available():
            torch.cuda.set_device(0)
        gpu = measure_reference_gpu(a, g, cams, torch.device("cuda", 0), a.steps, max(a.warmup, 3)) \
            if torch.cuda.is_available() else None
    if gpu is not None:
        # the reference rasterizer is CUDA-only: its own implementation of the path runs on the GPU
        val = mpix_all / (gpu["ms_per_step"] * 1e-3)
        line.update(value=val, ms_per_step=gpu["ms_per_step"], gpu_launches=None,
                    reference={"kind": "_ref", "what": "the reference's own CUDA extension (oracle/_ref, compiled "
                               "from its unmodified sources for sm_100), raw entry points, same scene / cameras / "
                               "colours / upstream gradients, one GPU; plane descriptors precomputed (favours it)",
                               "stages_ms_per_step": gpu.get("stages")},
                    cpu_baseline={"value": val, "unit": "Mpix/s", "cores": 0, "kind": "reference",
                                  "sample": "whole workload on the GPU: the reference has no CPU implementation of "
                                            "this path (its rasterizer is CUDA-only)"},
                    e2e={"value": mpix_all / (gpu["e2e_ms_per_step"] * 1e-3), "unit": "Mpix/s",
                         "ms_per_step": gpu["e2e_ms_per_step"], "h2d_bytes_per_step": gpu["h2d_bytes_per_step"],
                         "d2h_bytes_per_step": gpu["d2h_bytes_per_step"]})
        print(json.dumps(line), flush=True)
        return
    # no GPU or no compiled reference: the CPU oracle port on the host cores, bounded sample
    times = []
    if a.workload == "cfg0":
        t, mpix, sample = cfg0_cpu_gloo(a.steps, a.warmup)
    else:
        for i in range(a.warmup + a.steps):
            dt, mpix, sample = cpu_step_sample(cfg, a.gaussians, cam_idx=0)
            if i >= a.warmup:
                times.append(dt)
        t = statistics.mean(times)
    val = mpix / t
    line.update(value=val, ms_per_step=t * 1e3, gpu_launches=0,
                reference={"kind": "port", "what": "CPU oracle port (the reference rasterizer is CUDA-only and its "
                           "compiled extension or a GPU is not available here)"},
                cpu_baseline={"value": val, "unit": "Mpix/s", "cores": cores, "kind": "port", "sample": sample},
                e2e={"value": val, "unit": "Mpix/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm
# ncu capture of one launch each, one camera of the default workload (GB moved / GB algorithmic)
NCU_BWD_TRAFFIC, NCU_BWD_ALGO = 1.80, 0.827
NCU_FWD_TRAFFIC, NCU_FWD_ALGO = 0.432, 0.348

ALGO_BYTES = {
    # algorithmic bytes per launch (API-boundary tensors touched once); HW = pixels of the locally rendered tiles
    "cgx_preprocess_fwd": lambda i: 115 * i["P"],
    "cgx_preprocess_bwd": lambda i: 148 * i["P"],
    # camera-batched preprocess over B cameras: parameters read once (44 B), per camera means2D 8 + depth 4 +
    # radius 4 + conic_opacity 16 = 32 B out (+20 B of plane descriptors); backward: parameters 44 B, per camera
    # radius 4 + dL/dmeans2D 8 + dL/dconic_opacity 16 = 28 B in (+20 B), parameter gradients 44 B out
    "cgx_preprocess_fwd_batched": lambda i: i["P"] * (44 + (52 if i["planes"] else 32) * i["B"]),
    "cgx_preprocess_bwd_batched": lambda i: i["P"] * (88 + (48 if i["planes"] else 28) * i["B"]),
    # row-driven owner backward: per returned row its columns, its index, 44 B of gathered parameters and 56 B of
    # partial sums; per Gaussian 56 B of sums and 28 B of parameters in, 44 B of gradients out
    "cgx_preprocess_bwd_rows": lambda i: i["rows"] * (4 * i["ncols"] + 4 + 44 + 56) + i["P"] * (56 + 28 + 44),
    "cgx_bin_count_scan": lambda i: 16 * i["P"],
    "cgx_emit_keys": lambda i: 20 * i["P"] + 12 * i["R"],
    "cgx_sort_pairs": lambda i: i["R"] * (8 + 24 * ((i["bits"] + 7) // 8)),
    "cgx_tile_ranges": lambda i: 8 * i["R"] + 8 * i["T"],
    "cgx_render_fwd": lambda i: 60 * i["R"] + 48 * i["HW"],
    "cgx_render_bwd": lambda i: 60 * i["R"] + 60 * i["HW"] + 76 * i["P"],
}

# DRAM bytes moved per algorithmic byte of the two blending kernels: dram__bytes_read.sum + dram__bytes_write.sum of
# ONE launch captured with ncu on one camera of the default workload (the bench cannot run under a profiler), scaled
# to the run's launches by their algorithmic bytes.
DRAM_TRAFFIC_PER_ALGO_BYTE = {"cgx_render_bwd": NCU_BWD_TRAFFIC / NCU_BWD_ALGO, "cgx_render_fwd": NCU_FWD_TRAFFIC / NCU_FWD_ALGO}

# ncu counters of one launch of each blending kernel on one camera of the default workload (the same captures)
NCU_PIPE_COUNTERS = {
    "cgx_render_bwd": {"issue_active_pct": 67.7, "pipe_fma_pct": 32.4, "dram_throughput_pct": 17.9,
                       "warp_instructions": 0.949e9},
    "cgx_render_fwd": {"issue_active_pct": 78.4, "pipe_fma_pct": 35.2, "dram_throughput_pct": 9.9,
                       "warp_instructions": 0.470e9},
}

# FP32 instruction issue peak: 148 SMs x 128 FP32 lanes x 1.965 GHz (one FMA = one instruction)
FP32_PEAK_THREAD_INSTR_PER_S = 148 * 128 * 1.965e9


_local_pixels = {}


def resolve_info(info):
    """Turn the tensors a stage left in its info record into numbers (called after the run has been synchronised):
    `local` (bool tile mask) -> HW = pixels of local tiles; per-tile counters -> their sums."""
    if info is None:
        return None
    out = dict(info)
    local = out.pop("local", None)
    if local is not None:
        key = (local.data_ptr(), local._version, tuple(local.shape))
        if key not in _local_pixels:
            _local_pixels[key] = int(local.sum().item()) * 256
        out["HW"] = min(out["HW"], _local_pixels[key])
    for k in ("n_consider", "n_contrib"):
        t = out.pop(k, None)
        if t is not None:
            out[k + "_sum"] = int(t.sum(dtype=torch.int64).item())
    return out


def multi_gpu_parity(dev, rank, world):
    """Correctness of the distributed step, recorded beside its speed: a reduced scene (200k Gaussians, world+1
    cameras at 640x480, so that at least one camera is split between two ranks) through the same TrainingStep on all
    ranks, against the single-GPU step of the same scene on rank 0.  Returns the parity record (rank 0) or None."""
    import torch.distributed as dist

    from cgx import runtime as RT
    from cgx import synthetic as S

    n, res = 200_000, (640, 480)
    g, cams = S.config(2, n_gaussians=n, n_cameras=world + 1, res=res)
    step = RT.TrainingStep(g, cams, dev, rank=rank, world_size=world)
    step.run()
    strategies = step._strategies
    split = sum(1 for s in strategies if len(s.gpu_ids) > 1)
    transport = step.exchange_stats().get("transport")
    names = ("means3D", "scales", "rotations", "opacities")
    # gather every rank's shard gradients and local radii on rank 0 (shards are i % world)
    full = {k: torch.zeros_like(g[k], device=dev) for k in names}
    for k in names:
        full[k][rank::world] = step.params[k].grad
        dist.all_reduce(full[k])
    radii = torch.zeros(len(cams), n, dtype=torch.int32, device=dev)
    m2g = torch.zeros(len(cams), n, 2, device=dev)
    have_m2 = False
    for c, (rad, m2) in enumerate(step.last):
        radii[c, rank::world] = rad
        if m2.grad is not None:
            m2g[c, rank::world] = m2.grad
            have_m2 = True
    dist.all_reduce(radii)
    dist.all_reduce(m2g)
    torch.cuda.synchronize()
    out = None
    if rank == 0:
        single = RT.TrainingStep(g, cams, dev, rank=0, world_size=1)
        single.run()
        torch.cuda.synchronize()

        def rel(a, b):
            return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))

        errs = {k: rel(full[k], single.params[k].grad) for k in names}
        if have_m2:     # owner-side screen-space gradients exist only when the rows are scattered into dense arrays
            errs["means2D"] = max(rel(m2g[c], single.last[c][1].grad) for c in range(len(cams)))
        out = {"grad_rel_l2_max": max(errs.values()), "grad_rel_l2": errs,
               "radii_equal": all(bool(torch.equal(radii[c], single.last[c][0])) for c in range(len(cams))),
               "split_cameras": split, "transport": transport,
               "owner_backward": "row-driven, inside the exchange's backward" if not have_m2 else "dense cotangents",
               "case": f"{n} Gaussians, {len(cams)} cameras {res[0]}x{res[1]}, {world} ranks vs 1 GPU"}
        del single
    del step
    torch.cuda.empty_cache()
    dist.barrier()
    return out


def run_redistribute(a):
    """Times cgx.exchange.redistribute_rows on a model-state-shaped list of tensors; one JSON line with GB/s."""
    import torch.distributed as dist

    from cgx import exchange

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
    stdout_fd = os.dup(1)
    os.dup2(2, 1)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n = (a.gaussians or 6_000_000) // world
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    widths = {"anchor": 3, "offset": 30, "anchor_feat": 32, "opacity": 1, "scaling": 6, "rotation": 4}
    tensors = []
    for w in widths.values():                       # parameter, exp_avg, exp_avg_sq
        tensors += [torch.randn(n, w, device=dev, generator=gen) for _ in range(3)]
    tensors += [torch.randint(0, 6, (n, 1), device=dev, dtype=torch.int32, generator=gen),
                torch.rand(n, device=dev, generator=gen)]
    row_bytes = sum(t[0].numel() * t.element_size() for t in tensors)
    # the reference's destination rule (scene/gaussian_model.py:1660-1662), applied to a shard that is NOT yet round-robin
    dest = (torch.arange(n, device=dev) + rank) % world

    def one():
        out, _ = exchange.redistribute_rows(tensors, dest)
        return out

    for _ in range(max(a.warmup, 3)):
        one()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        one()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    moved = n * world * row_bytes
    if rank == 0:
        line = {"metric": "anchor redistribution GB/s (rows x 916 B moved per second, whole job)",
                "value": moved / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "steps": a.steps,
                "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "u32", "data": "synthetic",
                "config": {"workload": "redistribute", "description": WORKLOADS["redistribute"][1],
                           "rows": n * world, "row_bytes": row_bytes, "tensors": len(tensors),
                           "rows_leaving_each_rank": n - n // world if world > 1 else 0},
                "gpu_launches": 4}
        sys.stdout.flush()
        os.dup2(stdout_fd, 1)
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    a = parse_args()
    if a.impl == "reference":
        run_reference_arm(a)
        return
    if a.workload == "redistribute":
        run_redistribute(a)
        return

    from cgx import synthetic as S
    from cgx import runtime as RT

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rasterizer has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    stdout_fd = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only, no multicast objects
        # libraries underneath (NCCL's version banner) write to file descriptor 1; the one JSON line must be alone
        # on stdout, so everything else goes to stderr until that line is printed
        sys.stdout.flush()
        stdout_fd = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
    assert world == a.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"

    cfg = WORKLOADS[a.workload][0]
    g, cams = S.config(cfg, n_gaussians=a.gaussians)
    if a.cameras:
        cams = cams[: a.cameras]
    step = RT.TrainingStep(g, cams, dev, rank=rank, world_size=world)
    if a.densification_stats or a.workload == "cfg4":
        step.enable_densification_stats()
    if a.render_streams is not None:
        step.render_streams = a.render_streams
    mpix = sum(c.W * c.H for c in cams) / 1e6
    n_scene = g["means3D"].shape[0]

    from diff_gaussian_rasterization import _C, _lib
    lib = _lib.lib()
    if a.render_variant is not None:
        lib.cgx_set_render_variant(a.render_variant)
    if a.sort_variant is not None:
        lib.cgx_set_sort_variant(a.sort_variant)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, join=None):
        """K steps bracketed by barrier+sync; device time by CUDA events; max over ranks.  `join`: called after the
        last step and before the closing event, to put that event behind work queued on other streams."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if join is not None:
            join()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- device-resident measurement
    sampler = ClockSampler(local_rank)
    if rank == 0 and not a.no_clocks:
        sampler.start()                 # samples cover warm-up and the timed region (both under load)
    for _ in range(max(a.warmup, 3)):
        step.run()
    launches0 = lib.cgx_launch_count()
    ms_total = timed(step.run, a.steps)
    launches = (lib.cgx_launch_count() - launches0) // a.steps
    ms_step = ms_total / a.steps
    # per-stage pass: the same K steps again with CUDA events around every library call and every camera on ONE
    # stream, so that a launch's duration is that of the kernel alone (with two camera streams launches of different
    # cameras overlap and their durations stretch).  `value` comes from the pass above, the stage table and the
    # roofline from this one.
    prof, stage_pass = [], None
    if not a.no_stage_events:
        streams_default, step.render_streams = step.render_streams, 1
        for _ in range(3):          # the allocator's pools are per stream: let the one-stream pass fill its own
            step.run()
        _C.PROFILE = []
        ms_stage_pass = timed(step.run, a.steps) / a.steps
        prof, _C.PROFILE = (_C.PROFILE or []), None
        step.render_streams = streams_default
        stage_pass = {"ms_per_step": ms_stage_pass, "render_streams": 1,
                      "render_streams_timed": streams_default if world == 1 else 1}
    clocks = sampler.stop() if rank == 0 else None

    # per-stage device time (events recorded on the launching stream during the timed region)
    stages = {}
    for name, e0, e1, info in prof:
        s = stages.setdefault(name, {"ms": 0.0, "launches": 0, "bytes": 0.0, "fp32": 0.0})
        s["ms"] += e0.elapsed_time(e1)
        s["launches"] += 1
        info = resolve_info(info)
        if info is not None and name in ALGO_BYTES:
            s["bytes"] += ALGO_BYTES[name](info)
        if info is not None and "n_consider_sum" in info:
            # useful FP32 work of the blending: ~10 instructions per (pixel, Gaussian) pair examined up to the
            # pixel's last contributor, ~11 more per pair that contributes; both sums are outputs of the operator
            s["fp32"] += 10.0 * info["n_consider_sum"] + 11.0 * info["n_contrib_sum"]
            s["pairs"] = s.get("pairs", 0.0) + info["n_consider_sum"]
            s["contrib"] = s.get("contrib", 0.0) + info["n_contrib_sum"]
    # the backward blend walks the same pairs as the forward launches of the same pass (one backward per forward):
    # ~10 instructions per pair examined (the alpha test), ~90 per pair that contributes (recurrences + 16 terms)
    if "cgx_render_bwd" in stages and stages.get("cgx_render_fwd", {}).get("pairs"):
        f, b = stages["cgx_render_fwd"], stages["cgx_render_bwd"]
        if f["launches"] == b["launches"]:
            b["fp32"] = 10.0 * f["pairs"] + 90.0 * f["contrib"]
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peak, peak_src = json.loads(peaks_path.read_text())["hbm_gbs"], "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    stage_out = {}
    for name, s in stages.items():
        gbs = s["bytes"] / (s["ms"] * 1e-3) / 1e9 if s["ms"] > 0 and s["bytes"] else None
        stage_out[name] = {"ms_per_step": s["ms"] / a.steps, "launches_per_step": s["launches"] / a.steps,
                           "algo_gbs": gbs, "frac_of_hbm_peak": gbs / peak if gbs else None}
        if s["fp32"] and s["ms"] > 0:
            rate = s["fp32"] / (s["ms"] * 1e-3)
            stage_out[name]["useful_fp32_thread_instr_per_s"] = rate
            stage_out[name]["frac_of_fp32_issue_peak"] = rate / FP32_PEAK_THREAD_INSTR_PER_S
    top = max(stages, key=lambda k: stages[k]["ms"]) if stages else None
    roofline = None
    if top:
        s = stages[top]
        ach = s["bytes"] / (s["ms"] * 1e-3) / 1e9
        per_launch = s["bytes"] / s["launches"]
        ratio = DRAM_TRAFFIC_PER_ALGO_BYTE.get(top)
        roofline = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "traffic": per_launch * ratio if ratio else None,
                    "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on "
                                       "one camera of this workload, scaled by algorithmic bytes") if ratio else None,
                    "algo_bytes_per_launch": per_launch, "peak_source": peak_src,
                    "avg_launch_ms": s["ms"] / s["launches"],
                    "fp32": {"useful_thread_instr_per_s": stage_out[top].get("useful_fp32_thread_instr_per_s"),
                             "frac_of_issue_peak": stage_out[top].get("frac_of_fp32_issue_peak"),
                             "peak_thread_instr_per_s": FP32_PEAK_THREAD_INSTR_PER_S,
                             "ncu": NCU_PIPE_COUNTERS.get(top)},
                    "measured_in": "per-stage pass (the K steps again, one stream, CUDA events around each launch)",
                    "note": "blending is instruction-issue bound, not HBM bound (see fp32.ncu); the HBM fraction is "
                            "reported because the contract asks for an HBM or tensor roofline"}
    # the fused pack kernels ARE the transport of the peer-to-peer exchange: bytes crossing NVLink / their time
    ex = step.exchange_stats()
    if ex and ex.get("transport") == "p2p":
        for key, stage in (("fwd", "cgx_local2j_pack_p2p_batched"), ("bwd", "cgx_pack_grad_rows_to")):
            if stage in stages and stages[stage]["ms"] > 0:
                ms = stages[stage]["ms"] / a.steps
                ex[f"{key}_kernel_ms"] = ms
                ex[f"{key}_gbs_per_rank"] = ex[f"bytes_sent_{key}"] / (ms * 1e-3) / 1e9

    # ---- end-to-end: host inputs copied in, result read back, every step
    e2e = None
    if not a.no_e2e:
        for _ in range(max(a.warmup, 3) + 2):       # the first calls also allocate the second buffer set
            step.run_e2e()
        ms_e2e = timed(step.run_e2e, a.steps, join=step.join_e2e) / a.steps
        e2e = {"value": mpix / (ms_e2e * 1e-3), "unit": "Mpix/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": step.h2d_bytes, "d2h_bytes_per_step": step.d2h_bytes}

    # ---- multi-GPU: correctness of the distributed step on a reduced scene (after the timed regions: its
    # allocations and collectives must not disturb them)
    parity = multi_gpu_parity(dev, rank, world) if world > 1 and not a.no_parity else None

    # ---- the reference's own CUDA extension on the same GPU, same workload (rank 0, N=1 only)
    ref_gpu = None
    if rank == 0 and world == 1 and not a.no_ref_gpu:
        ref_gpu = measure_reference_gpu(a, g, cams, dev, min(a.steps, 10), 3, e2e=False)

    # ---- CPU baseline (rank 0, N=1 only): bounded sample
    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        cores = os.cpu_count() or 1
        os.environ.setdefault("OMP_NUM_THREADS", str(cores))
        if a.workload == "cfg0":
            dt, mp, sample = cfg0_cpu_gloo(3, 1)
        else:
            dt, mp, sample = cpu_step_sample(cfg, a.cpu_sample_gaussians or a.gaussians, cam_idx=0)
        cpu = {"value": mp / dt, "unit": "Mpix/s", "cores": cores, "kind": "port", "sample": sample,
               "seconds": dt}

    if a.kernel_table:
        from torch.profiler import ProfilerActivity, profile

        barrier()
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                step.run()
            torch.cuda.synchronize()
        if rank == 0:
            print("per-kernel device time over 3 steps (torch.profiler, rank 0):", file=sys.stderr)
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=70),
                  file=sys.stderr, flush=True)

    # balancer: per-rank render time (forward + backward, ms) of the first and the last recorded step
    balancer = None
    if world > 1 and step.history is not None and step.history.history:
        def summary(entry):
            t = entry["all_gpu_running_time"]
            return {"iteration": entry["iteration"], "max_ms": max(t), "mean_ms": sum(t) / len(t),
                    "per_rank_ms": [round(x, 3) for x in t]}
        h = step.history.history
        balancer = {"recorded_steps": len(h), "first": summary(h[0]), "last": summary(h[-1]),
                    "division_pos_last": [c["division_pos"] for c in h[-1]["batched_camera_info"]]}

    if rank == 0:
        line = {
            "metric": "fwd+bwd Mpix/s", "value": mpix / (ms_step * 1e-3), "unit": "Mpix/s", "n_gpus": world,
            "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(a, cams, n_scene),
            "gaussian_views_per_s": n_scene * len(cams) / (ms_step * 1e-3),
            "roofline": roofline, "stages": stage_out, "stage_pass": stage_pass, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "exchange": ex, "balancer": balancer,
            "parity": parity, "ref_gpu": ref_gpu,
            "densification_stats": step.densification_summary(),
        }
        if stdout_fd is not None:
            sys.stdout.flush()
            os.dup2(stdout_fd, 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
