"""One data-parallel step of the hot path, as the reference's training loop drives it
(train_internal.py:166-265; gaussian_renderer/__init__.py:903-1308 and :1325-1572):

    per camera: preprocess_gaussians on the local Gaussian shard
    (world_size > 1) all-to-all of the screen-space records to the ranks that own the touched tile rows
    per (camera, local row band): render_gaussians
    backward of everything (render bwd -> reverse all-to-all -> preprocess bwd)

This module owns no arithmetic: it allocates tensors, calls the drop-in `diff_gaussian_rasterization` API and
`cgx.exchange`, and is what bench.py and the smoke check time.  Upstream gradients are fixed N(0,1) images.
"""
from __future__ import annotations

import torch

from diff_gaussian_rasterization import GaussianRasterizationSettings, GaussianRasterizer, _C

from . import synthetic as S


def make_cuda_args(rank=0, world_size=1, iteration=1):
    """The dict of strings the reference passes down to its C++ ops (gaussian_renderer/__init__.py:523-537)."""
    return {"mode": "train", "world_size": str(world_size), "global_rank": str(rank), "local_rank": str(rank),
            "mp_world_size": str(world_size), "mp_rank": str(rank), "log_folder": "/tmp", "log_interval": "250",
            "iteration": str(iteration), "zhx_debug": "False", "zhx_time": "False", "dist_global_strategy": "",
            "avoid_pixel_all2all": False, "stats_collector": {}}


class _AwaitEvent(torch.autograd.Function):
    """Identity whose backward makes the current stream wait for a CUDA event first: placed on a camera's rendered
    images, it holds that camera's backward pass until the upstream-gradient images it reads have arrived."""

    @staticmethod
    def forward(ctx, event, *tensors):
        ctx.event = event
        return tuple(t.view_as(t) for t in tensors)

    @staticmethod
    def backward(ctx, *grads):
        torch.cuda.current_stream().wait_event(ctx.event)
        return (None,) + grads


class TrainingStep:
    def __init__(self, g, cams, device, rank=0, world_size=1, seed=4242, transport=None):
        self.dev, self.rank, self.ws = device, rank, world_size
        self.transport = transport      # None: peer-to-peer inside an NCCL group, collective otherwise
        self.batched = True             # camera-batched preprocess (False: the reference's per-camera loop)
        # True: the per-camera render times of step t ride on the size-table all-gather of step t+1 (their CUDA
        # events have completed by then and that collective is read on the host anyway), so the balancer costs no
        # collective and no host synchronisation of its own; its heuristics then lag one step behind the
        # reference's, which gathers the times at the end of every step.
        self.lazy_balancer = True
        self._pending_stats = None
        self._copy_stream = None
        self._d2h_stream = None
        self._cot_events = None         # per camera: event after which its upstream-gradient images are on the device
        # True: gradients of the plane descriptors flow back to means3D / rotations (through the reverse exchange
        # when distributed: 19-float gradient rows), as in the reference's training graph
        self.plane_grads = True
        self.densify = None             # DensificationStats, updated after every step when enabled
        self.prefetch_counts = True     # start every camera's pair counting before the first host read of a count
        self.cams = cams
        # Gaussians are stored round-robin over ranks, like the reference's anchors (scene/gaussian_model.py:476-479)
        sel = slice(rank, None, world_size)
        self.host = {k: g[k][sel].contiguous().pin_memory() for k in ("means3D", "scales", "rotations", "opacities")}
        self.params = {k: v.to(device).requires_grad_(True) for k, v in self.host.items()}
        sh = g["sh"][sel].contiguous().to(device)
        self.sh_dummy = torch.empty(0, device=device)
        self.n_local = self.params["means3D"].shape[0]
        gen = torch.Generator().manual_seed(seed)
        self.settings, self.rgb, self.all_map, self.cot_host, self.cot = [], [], [], [], []
        for cam in cams:
            self.settings.append(GaussianRasterizationSettings(
                image_height=cam.H, image_width=cam.W, tanfovx=cam.tanfovx, tanfovy=cam.tanfovy,
                bg=torch.zeros(3, device=device), scale_modifier=1.0, viewmatrix=cam.viewmatrix.to(device),
                projmatrix=cam.projmatrix.to(device), sh_degree=3, campos=cam.campos.to(device), prefiltered=False,
                render_geo=True, debug=False))
            with torch.no_grad():
                self.rgb.append(self._colours(sh, cam))
            ch = [torch.randn(3, cam.H, cam.W, generator=gen), torch.randn(5, cam.H, cam.W, generator=gen),
                  torch.randn(1, cam.H, cam.W, generator=gen)]
            self.cot_host.append([c.pin_memory() for c in ch])
            self.cot.append([c.to(device) for c in ch])
        del sh
        self.grad_host = {k: torch.empty_like(v).pin_memory() for k, v in self.host.items()}
        self.h2d_bytes = sum(v.numel() * 4 for v in self.host.values()) + \
            sum(c.numel() * 4 for cs in self.cot_host for c in cs)
        self.d2h_bytes = sum(v.numel() * 4 for v in self.grad_host.values())
        self.iteration = 0
        self._exchange = {"bytes_sent_fwd": 0, "bytes_sent_bwd": 0, "ms": 0.0}
        self.last = None
        self.history = None
        if world_size > 1:
            from . import workload_division as WD

            self.ctx = WD.DivisionContext(image_height=cams[0].H, image_width=cams[0].W, rank=rank,
                                          world_size=world_size, bsz=len(cams), device=device)
            self.history = WD.DivisionStrategyHistoryFinal(cams, world_size, rank, ctx=self.ctx)

    def all_map_for(self, k, means3D, scales, rotations, radii):
        """Plane descriptors of the rows about to be rendered for camera k: one kernel each way, differentiable
        towards means3D and rotations as the reference's tensor code is (gaussian_renderer/__init__.py:1501-1518)."""
        from .plane_map import plane_map

        rs = self.settings[k]
        if not self.plane_grads:
            means3D, scales, rotations = means3D.detach(), scales.detach(), rotations.detach()
        return plane_map(means3D, scales, rotations, rs.viewmatrix, rs.campos, radii)

    def _colours(self, sh, cam):
        """View-dependent colours through the library's SH stage (degree 3), as activated RGB."""
        import ctypes as C

        from diff_gaussian_rasterization import _lib

        P = sh.shape[0]
        rgb = torch.empty(P, 3, device=self.dev)
        clamped = torch.empty(P, 3, dtype=torch.bool, device=self.dev)
        if P:
            cp = cam.campos.to(self.dev)
            _lib.check(_lib.lib().cgx_sh_to_rgb(P, 3, 16, self.params["means3D"].data_ptr(), cp.data_ptr(),
                                                sh.data_ptr(), rgb.data_ptr(), clamped.data_ptr(),
                                                _lib.current_stream_ptr()), "cgx_sh_to_rgb")
        return rgb

    # ------------------------------------------------------------------ single-GPU step
    _pipeline = None        # cgx.batched.Pipeline while an end-to-end step is in flight
    _e2e_sets = None        # two (parameters, upstream-gradient images) buffer sets that end-to-end steps alternate

    def _preprocess_all(self, args, planes=False):
        """Screen-space state of the local Gaussians for every camera of the batch (one launch).  With `planes`
        every camera's tuple ends with its differentiable plane descriptors (fused into the same launches when
        batched, the stand-alone op otherwise)."""
        from .batched import preprocess_gaussians_batched

        p = self.params
        if self.batched:
            return preprocess_gaussians_batched(p["means3D"], p["scales"], p["rotations"], self.sh_dummy,
                                                p["opacities"], self.settings, args, planes=planes,
                                                pipeline=self._pipeline)
        out = [GaussianRasterizer(s).preprocess_gaussians(p["means3D"], p["scales"], p["rotations"], self.sh_dummy,
                                                          p["opacities"], args) for s in self.settings]
        if planes:
            out = [t + (self.all_map_for(k, p["means3D"], p["scales"], p["rotations"], t[3]),)
                   for k, t in enumerate(out)]
        return out

    def _step_single(self):
        p = self.params
        args = make_cuda_args(self.rank, self.ws, self.iteration)
        outs, heads, grads = [], [], []
        screen = self._preprocess_all(args, planes=self.plane_grads)
        if self.prefetch_counts:
            for k, cam in enumerate(self.cams):     # every camera's pair count is on its way before the first read
                _C.prefetch_num_rendered(cam.H, cam.W, screen[k][0], screen[k][3],
                                         self._all_local((cam.H + 15) // 16, (cam.W + 15) // 16), depths=screen[k][4])
        # Cameras are independent until the parameter gradients are summed: they alternate between `render_streams`
        # CUDA streams, so that the binning / sorting of one camera (memory- and launch-bound) runs beside the
        # blending of another (instruction-bound).  Autograd runs each camera's backward on the stream of its forward.
        main = torch.cuda.current_stream()
        streams = self._streams(main)
        for s in streams:
            s.wait_stream(main)
        for k, cam in enumerate(self.cams):
            with torch.cuda.stream(streams[k % len(streams)]):
                rast = GaussianRasterizer(self.settings[k])
                means2D, _, conic_opacity, radii, depths = screen[k][:5]
                means2D.retain_grad()          # the densifier reads means2D.grad
                TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
                local = self._all_local(TY, TX)
                means2D_abs = torch.zeros(self.n_local, 3, device=self.dev, requires_grad=True)
                all_map = screen[k][5] if self.plane_grads else \
                    self.all_map_for(k, p["means3D"], p["scales"], p["rotations"], radii)
                color, n_render, n_consider, n_contrib, observe, out_all_map, plane_depth = rast.render_gaussians(
                    means2D, means2D_abs, conic_opacity, self.rgb[k], all_map, depths, radii, local, None, args)
                if self._cot_events is not None and k in self._cot_events:
                    color, out_all_map, plane_depth = _AwaitEvent.apply(self._cot_events[k], color, out_all_map,
                                                                        plane_depth)
                heads += [color, out_all_map, plane_depth]
                grads += self.cot[k]
                outs.append((radii, means2D))
        for s in streams:
            main.wait_stream(s)
        torch.autograd.backward(heads, grads)      # one backward over the batch, as one loss.backward() upstream
        for s in streams:                          # the backward kernels of the side streams precede whatever follows
            main.wait_stream(s)
        self.last = outs

    render_streams = 2      # cameras of the single-GPU step alternate between that many CUDA streams (1: one stream)
    _side_streams = None

    def _streams(self, main):
        if self.render_streams <= 1:
            return [main]
        if self._side_streams is None or len(self._side_streams) != self.render_streams:
            self._side_streams = [torch.cuda.Stream(device=self.dev) for _ in range(self.render_streams)]
        return self._side_streams

    _local_cache = {}

    def _all_local(self, TY, TX):
        key = (TY, TX, self.dev)
        if key not in self._local_cache:
            self._local_cache[key] = torch.ones(TY, TX, dtype=torch.bool, device=self.dev)
        return self._local_cache[key]

    def enable_densification_stats(self):
        from .densification import DensificationStats

        self.densify = DensificationStats(self.n_local, self.dev)

    def densification_summary(self):
        """Small host-side digest of the accumulated statistics (one synchronising read; call outside timed code)."""
        if self.densify is None:
            return None
        d = self.densify
        seen = d.denom > 0
        return {"gaussians_seen": int(seen.sum().item()), "visits": float(d.denom.sum().item()),
                "mean_grad_norm": float(d.mean_gradient()[seen].mean().item()) if bool(seen.any()) else 0.0,
                "max_radius": int(d.max_radii2D.max().item())}

    def run(self):
        self.iteration += 1
        for v in self.params.values():
            v.grad = None
        if self.ws == 1:
            self._step_single()
        else:
            self._step_distributed()
            if not self.lazy_balancer:
                self.finish_balancer()
        if self.densify is not None:
            self.densify.update_batch(self.last)
        return self.params

    # ------------------------------------------------------------------ multi-GPU step
    owner_backward = True   # fold the owner's preprocess backward into the exchange's backward when nothing reads
                            # the owner-side screen-space gradients
    def forward_only(self):
        """The distributed forward pass without a graph (an evaluation render, or the reference's second exchange
        for the nearest-view cameras, gaussian_renderer/__init__.py:1026,1439-1458): preprocess, exchange, render of
        the local tile rows; no reverse exchange follows.  Returns the rendered (color, all_map, plane_depth) per
        camera (None where this rank renders nothing)."""
        with torch.no_grad():
            return self._step_distributed(backward=False)

    def _step_distributed(self, backward=True):
        from . import exchange
        from . import workload_division as WD

        p = self.params
        self.ctx.iteration = self.iteration
        strategies, _ = WD.start_strategy_final(self.cams, self.history, ctx=self.ctx)
        rasts = [GaussianRasterizer(s) for s in self.settings]
        args = [make_cuda_args(self.rank, self.ws, self.iteration) for _ in self.cams]
        # Plane descriptors: computed by the owner inside the preprocess launch and sent instead of the 3-D
        # parameters when the exchange stores straight into peer memory; otherwise the 3-D parameters travel
        # (differentiably) and the descriptors are rebuilt on the receiver, as the reference does.
        fused = self.plane_grads and self.batched and \
            exchange._pick_transport(self.transport, None, self.dev, exchange.default_backend()) == "p2p"
        # With the fused record form and no consumer of the owner-side screen-space gradients (the densifier reads
        # means2D.grad), the preprocess runs outside the graph and the exchange's backward does its backward too.
        owner = None
        if fused and backward and torch.is_grad_enabled() and self.owner_backward and self.densify is None:
            with torch.no_grad():
                pre = self._preprocess_all(args[0], planes=True)
            owner = dict(params=(p["means3D"], p["scales"], p["rotations"], p["opacities"]), settings=self.settings,
                         pipeline=self._pipeline)
        else:
            pre = self._preprocess_all(args[0], planes=fused)
        screen, keep = [], []
        for k in range(len(self.cams)):
            means2D, _, conic_opacity, radii, depths = pre[k][:5]
            if means2D.requires_grad:
                means2D.retain_grad()
            keep.append((radii, means2D))
            if fused:
                screen.append((means2D, self.rgb[k], conic_opacity, radii, depths, pre[k][5]))
                continue
            m3, sc, rot = p["means3D"], p["scales"], p["rotations"]
            if not self.plane_grads:
                m3, sc, rot = m3.detach(), sc.detach(), rot.detach()
            screen.append((means2D, self.rgb[k], conic_opacity, radii, depths, m3, sc, rot))
        pending, times = self._pending_stats, None
        if backward and self.lazy_balancer and pending is not None:
            times = WD.local_running_times(pending[0], pending[1], ctx=self.ctx)
        (m2, rgb, co, rad, dep, m3, sc, rot, sizes, sent, send_index, stats) = \
            exchange.all_to_all_communication_final(rasts, screen, args, strategies, transport=self.transport,
                                                    piggyback=times, planes=fused, owner=owner)
        if times is not None:
            WD.finish_strategy_final(self.cams, self.history, pending[0], pending[1], ctx=self.ctx,
                                     gathered_times=stats["piggyback"])
        self._exchange.update(bytes_sent_fwd=stats["bytes_sent_fwd"], bytes_sent_bwd=stats["bytes_sent_bwd"],
                              transport=stats["transport"], rows_sent=stats["rows_sent"],
                              record="plane descriptors (16 floats fwd, 14 bwd)" if fused
                              else "3-D parameters (21 floats fwd, 19 or 9 bwd)")
        heads, grads = [], []
        images = [None] * len(self.cams)
        if self.prefetch_counts:
            for k, strat in enumerate(strategies):
                local = strat.get_compute_locally()
                if local is not None and m2[k].shape[0] >= 10:
                    _C.prefetch_num_rendered(self.cams[k].H, self.cams[k].W, m2[k], rad[k], local, depths=dep[k])
        for k, strat in enumerate(strategies):
            local = strat.get_compute_locally()
            n_rows = m2[k].shape[0]
            if local is None or n_rows < 10:
                args[k]["stats_collector"].update(forward_render_time=0.0, backward_render_time=0.0)
                continue
            all_map = m3[k] if fused else self.all_map_for(k, m3[k], sc[k], rot[k], rad[k])
            m2abs = torch.zeros(n_rows, 3, device=self.dev, requires_grad=True)
            color, _, _, _, _, out_all_map, plane_depth = rasts[k].render_gaussians(
                m2[k], m2abs, co[k], rgb[k], all_map, dep[k], rad[k], local, None, args[k])
            if self._cot_events is not None and k in self._cot_events:
                color, out_all_map, plane_depth = _AwaitEvent.apply(self._cot_events[k], color, out_all_map,
                                                                    plane_depth)
            heads += [color, out_all_map, plane_depth]
            grads += self.cot[k]
            images[k] = (color, out_all_map, plane_depth)
        if not backward:
            return images
        if not heads:
            # nothing to render on this rank, but the reverse exchange is collective: keep its node in the graph
            heads.append(m2[0].sum() * 0.0)
            grads.append(torch.zeros((), device=self.dev))
        torch.autograd.backward(heads, grads)
        self.last = keep
        self._strategies = strategies
        self._stats = [a["stats_collector"] for a in args]
        self._pending_stats = (self._strategies, self._stats) if self.lazy_balancer else None

    def finish_balancer(self):
        """Feed measured render times back into the division heuristics (one tiny all-gather)."""
        if self.ws > 1:
            self._finish(self._strategies, self._stats)

    def _finish(self, strategies, stats):
        from . import workload_division as WD

        WD.finish_strategy_final(self.cams, self.history, strategies, stats, ctx=self.ctx)

    def run_e2e(self, chunks=4):
        """The same step with its host-side inputs copied in from pinned memory (Gaussian parameters and the
        upstream-gradient images) and the parameter gradients read back, all inside the caller's timed region.

        Copies run on a second stream and overlap the kernels where the data flow allows it: the parameters arrive in
        `chunks` pieces and the batched preprocess starts on each piece as it lands; the upstream-gradient images,
        first read by the backward pass, are copied beside the forward pass in the order the backward consumes them,
        and each camera's backward waits for its own images only; the parameter gradients leave piece by piece
        behind the chunks of the batched preprocess backward, on a stream of their own: the call returns without
        waiting for them, so that the read-back of step t (device to host) runs beside the uploads of step t + 1
        (host to device) when steps follow each other.  Parameters and images land in one of two buffer sets that
        alternate between calls, so the uploads of a call do not wait for the kernels of the call before it: they
        run beside its backward pass (the host is free as soon as that pass is queued).  `finish_e2e()` waits for
        everything; `grad_host` is complete after it.  `self.params` names the set of the latest call."""
        from .batched import Pipeline, chunk_bounds

        main = torch.cuda.current_stream()
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.dev)
            self._d2h_stream = torch.cuda.Stream(device=self.dev)
        copy, down = self._copy_stream, self._d2h_stream
        # piecewise gradient read-back needs the batched preprocess backward to be the ONLY producer of the parameter
        # gradients: true when the plane descriptors are fused into it (or switched off)
        from . import exchange
        fused = self.ws == 1 or not self.plane_grads or \
            exchange._pick_transport(self.transport, None, self.dev, exchange.default_backend()) == "p2p"
        pipelined = self.batched and chunks > 1 and fused
        bounds = chunk_bounds(self.n_local, chunks if pipelined else 1)
        names = ("means3D", "scales", "rotations", "opacities")
        # Two sets of device buffers alternate between steps: the uploads of step t + 1 wait only for the kernels of
        # step t - 1 (the last user of their set) and so run beside the kernels of step t.
        if self._e2e_sets is None:
            with torch.no_grad():
                other = ({k: v.detach().clone().requires_grad_(True) for k, v in self.params.items()},
                         [[c.clone() for c in cs] for cs in self.cot])
            self._e2e_sets = [(self.params, self.cot), other]
            self._e2e_free = [None, None]
            self._e2e_count = 0
        which = self._e2e_count & 1
        self._e2e_count += 1
        self.params, self.cot = self._e2e_sets[which]
        with torch.no_grad():
            if self._e2e_free[which] is not None:
                copy.wait_event(self._e2e_free[which])   # the step before last has finished with this set
            else:
                copy.wait_stream(main)
            ready = []
            with torch.cuda.stream(copy):
                for lo, hi in bounds:
                    for k in names:
                        self.params[k][lo:hi].copy_(self.host[k][lo:hi], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy)
                    ready.append(ev)
                # the backward pass walks the cameras last to first, so their images are sent in that order and
                # each camera's backward waits for its own images only
                mine = self._my_cameras()
                events = {}
                for k in reversed(mine):
                    for dst, src in zip(self.cot[k], self.cot_host[k]):
                        dst.copy_(src, non_blocking=True)
                    events[k] = torch.cuda.Event()
                    events[k].record(copy)
                self._cot_events = events
            self.h2d_bytes = sum(v.numel() * 4 for v in self.host.values()) + \
                sum(c.numel() * 4 for k in mine for c in self.cot_host[k])

        def gradients_out(i, lo, hi, grads):
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            with torch.cuda.stream(down):
                down.wait_event(ev)
                for k, g in zip(names, grads):
                    g.record_stream(down)
                    self.grad_host[k][lo:hi].copy_(g[lo:hi], non_blocking=True)

        if pipelined:
            self._pipeline = Pipeline(bounds, ready=ready, done=gradients_out)
        else:
            main.wait_event(ready[-1])
        try:
            self.run()
        finally:
            self._pipeline = None
            self._cot_events = None
        self._e2e_free[which] = torch.cuda.Event()
        self._e2e_free[which].record(main)
        if not pipelined:
            down.wait_stream(main)
            with torch.cuda.stream(down):
                for k, v in self.params.items():
                    v.grad.record_stream(down)
                    self.grad_host[k].copy_(v.grad, non_blocking=True)
        return self.grad_host

    def join_e2e(self):
        """Make the current stream wait for the copies of the end-to-end steps queued so far (no host wait): an
        event recorded on the current stream afterwards lies behind the last gradient's arrival on the host."""
        for s in (self._copy_stream, self._d2h_stream):
            if s is not None:
                torch.cuda.current_stream().wait_stream(s)

    def finish_e2e(self):
        """Wait for the copies and kernels of the end-to-end steps queued so far."""
        for s in (self._copy_stream, self._d2h_stream):
            if s is not None:
                s.synchronize()
        torch.cuda.current_stream().synchronize()

    def _my_cameras(self):
        """Cameras (part of) which this rank renders: all of them on one GPU, the balancer's choice otherwise."""
        if self.ws == 1:
            return list(range(len(self.cams)))
        from . import workload_division as WD

        strategies, _ = WD.start_strategy_final(self.cams, self.history, ctx=self.ctx)
        return [k for k, s in enumerate(strategies) if self.rank in s.gpu_ids]

    def exchange_stats(self):
        return None if self.ws == 1 else dict(self._exchange)
