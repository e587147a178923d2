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

from diff_gaussian_rasterization import _lib

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


def _ptrs(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


class _PreprocessBatched(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means3D, scales, rotations, opacities, settings, cuda_args):
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
        if P:
            cams, keep = _cams(settings)
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().cgx_preprocess_fwd_batched(
                    P, B, means3D.data_ptr(), scales.data_ptr(), float(settings[0].scale_modifier),
                    rotations.data_ptr(), opacities.data_ptr(), cams, _ptrs(m2), _ptrs(dep), _ptrs(rad), _ptrs(co),
                    _lib.current_stream_ptr()), "cgx_preprocess_fwd_batched")
        ctx.settings = settings
        ctx.save_for_backward(means3D, scales, rotations, *rad)
        flat = []
        for b in range(B):
            flat += [m2[b], co[b], rad[b], dep[b]]
        ctx.mark_non_differentiable(*rad, *dep)
        return tuple(flat)

    @staticmethod
    def backward(ctx, *grads):
        means3D, scales, rotations, *rad = ctx.saved_tensors
        settings = ctx.settings
        P, dev = means3D.shape[0], means3D.device
        d_means = torch.empty(P, 3, device=dev)
        d_scales = torch.empty(P, 3, device=dev)
        d_rot = torch.empty(P, 4, device=dev)
        d_op = torch.empty(P, 1, device=dev)
        use, g_m2, g_co = [], [], []
        for b in range(len(settings)):
            gm, gc = grads[4 * b], grads[4 * b + 1]
            if gm is None and gc is None:
                continue                      # this camera received no cotangent: it contributes nothing
            use.append(b)
            g_m2.append(gm.contiguous() if gm is not None else torch.zeros(P, 2, device=dev))
            g_co.append(gc.contiguous() if gc is not None else torch.zeros(P, 4, device=dev))
        if P and use:
            cams, keep = _cams([settings[b] for b in use])
            with torch.cuda.device(dev):
                _lib.check(_lib.lib().cgx_preprocess_bwd_batched(
                    P, len(use), means3D.data_ptr(), scales.data_ptr(), float(settings[0].scale_modifier),
                    rotations.data_ptr(), cams, _ptrs([rad[b] for b in use]), _ptrs(g_m2), _ptrs(g_co),
                    d_means.data_ptr(), d_scales.data_ptr(), d_rot.data_ptr(), d_op.data_ptr(),
                    _lib.current_stream_ptr()), "cgx_preprocess_bwd_batched")
        else:
            for t in (d_means, d_scales, d_rot, d_op):
                t.zero_()
        return d_means, d_scales, d_rot, d_op, None, None


def preprocess_gaussians_batched(means3D, scales, rotations, shs, opacities, raster_settings_list, cuda_args=None):
    """One (means2D, rgb, conic_opacity, radii, depths) tuple per camera, as the per-camera operator returns them
    (``rgb`` is the shared all-zero tensor the per-camera operator also returns: SH evaluation is compiled out)."""
    settings = list(raster_settings_list)
    flat = _PreprocessBatched.apply(means3D, scales, rotations, opacities, settings, cuda_args)
    rgb = torch.zeros(means3D.shape[0], 3, device=means3D.device)
    return [(flat[4 * b], rgb, flat[4 * b + 1], flat[4 * b + 2], flat[4 * b + 3]) for b in range(len(settings))]
