"""Camera-batched form of ``GaussianRasterizer.preprocess_gaussians``.

The reference's caller preprocesses its local Gaussians once per camera of the batch in a Python loop
(gaussian_renderer/__init__.py:966-1023).  Here the loop is one kernel launch: parameters are read once and
projected into all cameras; in the backward they are read once and the parameter gradients come out already
summed over the cameras (the reference leaves that sum to autograd's gradient accumulation).  Per camera the
outputs are bit-identical to the per-camera operator.
"""
from __future__ import annotations

import ctypes as C

import torch

from diff_gaussian_rasterization import _C, _lib

MAX_CAMS = 16


class _Camera(C.Structure):
    _fields_ = [("viewmatrix", C.c_void_p), ("projmatrix", C.c_void_p), ("tanfovx", C.c_float),
                ("tanfovy", C.c_float), ("W", C.c_int), ("H", C.c_int)]


def _cams(settings):
    arr = (_Camera * len(settings))()
    keep = []
    for b, rs in enumerate(settings):
        v, p = rs.viewmatrix.contiguous(), rs.projmatrix.contiguous()
        if not v.is_cuda or not p.is_cuda:
            raise RuntimeError("camera matrices must be CUDA tensors")
        keep += [v, p]
        arr[b].viewmatrix, arr[b].projmatrix = v.data_ptr(), p.data_ptr()
        arr[b].tanfovx, arr[b].tanfovy = float(rs.tanfovx), float(rs.tanfovy)
        arr[b].W, arr[b].H = int(rs.image_width), int(rs.image_height)
    return arr, keep


def _ptrs(tensors, row0=0):
    """Host array of device pointers to row `row0` of each (contiguous, row-major) tensor; None entries stay null."""
    return (C.c_void_p * len(tensors))(*[None if t is None else t.data_ptr() + row0 * t.stride(0) * t.element_size()
                                         for t in tensors])


def _row(t, row0):
    return t.data_ptr() + row0 * t.stride(0) * t.element_size()


def chunk_bounds(P, chunks):
    """[(lo, hi)] covering range(P) in `chunks` pieces whose starts are multiples of 256 rows (whole CTAs, and every
    row offset stays 16-byte aligned for the vectorised loads)."""
    chunks = max(1, int(chunks))
    per_chunk = -(-P // chunks)                               # ceil
    step = max(256, (per_chunk + 255) // 256 * 256)
    out, lo = [], 0
    while lo < P:
        out.append((lo, min(P, lo + step)))
        lo += step
    return out or [(0, 0)]


class Pipeline:
    """Optional hooks that let a caller overlap host<->device copies with the two launches, chunk by chunk over the
    Gaussians: `bounds` = chunk_bounds(P, n); `ready[i]` = CUDA event after which chunk i of the parameters may be
    read (the forward waits for it on the launching stream); `done(i, lo, hi, grads)` is called right after chunk i
    of the backward has been queued, with the four full gradient tensors (rows lo:hi are final once the launch
    completes)."""

    def __init__(self, bounds, ready=None, done=None):
        self.bounds, self.ready, self.done = bounds, ready, done


class _PreprocessBatched(torch.autograd.Function):
    """Outputs per camera: means2D, conic_opacity, radii, depths[, all_map when `planes`]."""

    @staticmethod
    def forward(ctx, means3D, scales, rotations, opacities, settings, cuda_args, planes, pipeline=None):
        if means3D.ndim != 2 or means3D.shape[1] != 3:
            raise RuntimeError("means3D must have dimensions (num_points, 3)")
        if not means3D.is_cuda:
            raise RuntimeError("means3D must be a CUDA tensor (this rasterizer has no CPU path)")
        B, P, dev = len(settings), means3D.shape[0], means3D.device
        if not 1 <= B <= MAX_CAMS:
            raise RuntimeError(f"between 1 and {MAX_CAMS} cameras per batched call")
        means3D, scales, rotations, opacities = (t.contiguous() for t in (means3D, scales, rotations, opacities))
        m2 = [torch.empty(P, 2, device=dev) for _ in range(B)]
        dep = [torch.empty(P, device=dev) for _ in range(B)]
        rad = [torch.empty(P, dtype=torch.int32, device=dev) for _ in range(B)]
        co = [torch.empty(P, 4, device=dev) for _ in range(B)]
        am = [torch.empty(P, 5, device=dev) for _ in range(B)] if planes else []
        if P:
            cams, keep = _cams(settings)
            campos = [rs.campos.contiguous() for rs in settings] if planes else None
            bounds = pipeline.bounds if pipeline is not None else [(0, P)]
            with torch.cuda.device(dev):
                for i, (lo, hi) in enumerate(bounds):
                    if pipeline is not None and pipeline.ready is not None:
                        torch.cuda.current_stream().wait_event(pipeline.ready[i])
                    _C._call("cgx_preprocess_fwd_batched", _lib.lib().cgx_preprocess_fwd_batched_planes,
                        hi - lo, B, _row(means3D, lo), _row(scales, lo), float(settings[0].scale_modifier),
                        _row(rotations, lo), _row(opacities, lo), cams, _ptrs(campos) if planes else None,
                        _ptrs(m2, lo), _ptrs(dep, lo), _ptrs(rad, lo), _ptrs(co, lo),
                        _ptrs(am, lo) if planes else None, _lib.current_stream_ptr(),
                        info=dict(P=hi - lo, B=B, planes=planes))
        ctx.settings, ctx.planes, ctx.pipeline = settings, planes, pipeline
        ctx.save_for_backward(means3D, scales, rotations, *rad)
        flat = []
        for b in range(B):
            flat += [m2[b], co[b], rad[b], dep[b]] + ([am[b]] if planes else [])
        ctx.mark_non_differentiable(*rad, *dep)
        return tuple(flat)

    @staticmethod
    def backward(ctx, *grads):
        means3D, scales, rotations, *rad = ctx.saved_tensors
        settings, planes = ctx.settings, ctx.planes
        n_out = 5 if planes else 4
        P, dev = means3D.shape[0], means3D.device
        d_means = torch.empty(P, 3, device=dev)
        d_scales = torch.empty(P, 3, device=dev)
        d_rot = torch.empty(P, 4, device=dev)
        d_op = torch.empty(P, 1, device=dev)
        use, g_m2, g_co, g_am = [], [], [], []
        for b in range(len(settings)):
            gm, gc = grads[n_out * b], grads[n_out * b + 1]
            ga = grads[n_out * b + 4] if planes else None
            if gm is None and gc is None and ga is None:
                continue                      # this camera received no cotangent: it contributes nothing
            use.append(b)
            g_m2.append(gm.contiguous() if gm is not None else torch.zeros(P, 2, device=dev))
            g_co.append(gc.contiguous() if gc is not None else torch.zeros(P, 4, device=dev))
            g_am.append(ga.contiguous() if ga is not None else None)
        if P and use:
            cams, keep = _cams([settings[b] for b in use])
            with_planes = planes and any(g is not None for g in g_am)
            campos = [settings[b].campos.contiguous() for b in use] if with_planes else None
            pipeline = ctx.pipeline
            bounds = pipeline.bounds if pipeline is not None else [(0, P)]
            with torch.cuda.device(dev):
                for i, (lo, hi) in enumerate(bounds):
                    _C._call("cgx_preprocess_bwd_batched", _lib.lib().cgx_preprocess_bwd_batched_planes,
                        hi - lo, len(use), _row(means3D, lo), _row(scales, lo), float(settings[0].scale_modifier),
                        _row(rotations, lo), cams, _ptrs(campos) if with_planes else None,
                        _ptrs([rad[b] for b in use], lo), _ptrs(g_m2, lo), _ptrs(g_co, lo),
                        _ptrs(g_am, lo) if with_planes else None,
                        _row(d_means, lo), _row(d_scales, lo), _row(d_rot, lo), _row(d_op, lo),
                        _lib.current_stream_ptr(), info=dict(P=hi - lo, B=len(use), planes=with_planes))
                    if pipeline is not None and pipeline.done is not None:
                        pipeline.done(i, lo, hi, (d_means, d_scales, d_rot, d_op))
        else:
            for t in (d_means, d_scales, d_rot, d_op):
                t.zero_()
        return d_means, d_scales, d_rot, d_op, None, None, None, None


def preprocess_gaussians_batched(means3D, scales, rotations, shs, opacities, raster_settings_list, cuda_args=None,
                                 planes=False, pipeline=None):
    """One (means2D, rgb, conic_opacity, radii, depths) tuple per camera, as the per-camera operator returns them
    (``rgb`` is the shared all-zero tensor the per-camera operator also returns: SH evaluation is compiled out).

    ``planes=True`` appends the camera's plane descriptors ``all_map`` (P,5) to each tuple: what the reference's
    caller builds after preprocessing (gaussian_renderer/__init__.py:1501-1518) comes out of the same launch, and
    its gradient towards means3D / rotations is folded into the same backward launch (see cgx.plane_map for the
    stand-alone op).  ``pipeline`` (a `Pipeline`) splits both launches into chunks of Gaussians so that a caller
    can overlap its host-to-device parameter copies and device-to-host gradient copies with them."""
    settings = list(raster_settings_list)
    flat = _PreprocessBatched.apply(means3D, scales, rotations, opacities, settings, cuda_args, bool(planes), pipeline)
    rgb = torch.zeros(means3D.shape[0], 3, device=means3D.device)
    n = 5 if planes else 4
    return [(flat[n * b], rgb, flat[n * b + 1], flat[n * b + 2], flat[n * b + 3]) + ((flat[n * b + 4],) if planes else ())
            for b in range(len(settings))]
