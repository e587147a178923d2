"""PGSR per-Gaussian plane descriptor ``all_map`` = [normal in camera space (3), 1, plane distance] as a
differentiable op: what the reference's caller builds with a dozen tensor operations right before
``render_gaussians`` (gaussian_renderer/__init__.py:1501-1518) is one kernel forward and one kernel backward here.

Gradients flow to ``means3D`` (through the distance) and to the raw quaternions (through the chosen rotation
column and ``normalize``); ``scales`` only select the column and receive none, exactly as in the reference's graph.
Rows with ``radii <= 0`` (never rasterized) are zero in both directions.
"""
from __future__ import annotations

import torch

from diff_gaussian_rasterization import _lib


class _PlaneMap(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means3D, scales, rotations, radii, viewmatrix, campos):
        for name, t in (("means3D", means3D), ("scales", scales), ("rotations", rotations),
                        ("viewmatrix", viewmatrix), ("campos", campos)):
            if not t.is_cuda or t.dtype != torch.float32:
                raise RuntimeError(f"plane_map: {name} must be a float32 CUDA tensor (no CPU path)")
        means3D, scales, rotations = means3D.contiguous(), scales.contiguous(), rotations.contiguous()
        viewmatrix, campos = viewmatrix.contiguous(), campos.contiguous()
        radii = None if radii is None else radii.contiguous()
        P = means3D.shape[0]
        out = torch.empty(P, 5, device=means3D.device, dtype=torch.float32)
        if P:
            _lib.check(_lib.lib().cgx_all_map_fwd(P, means3D.data_ptr(), scales.data_ptr(), rotations.data_ptr(),
                                                  None if radii is None else radii.data_ptr(), viewmatrix.data_ptr(),
                                                  campos.data_ptr(), out.data_ptr(), _lib.current_stream_ptr()),
                       "cgx_all_map_fwd")
        ctx.save_for_backward(means3D, scales, rotations, viewmatrix, campos)
        ctx.radii = radii
        return out

    @staticmethod
    def backward(ctx, g):
        means3D, scales, rotations, viewmatrix, campos = ctx.saved_tensors
        P = means3D.shape[0]
        d_means = torch.empty_like(means3D)
        d_rot = torch.empty_like(rotations)
        if P:
            g = g.contiguous()
            _lib.check(_lib.lib().cgx_all_map_bwd(P, means3D.data_ptr(), scales.data_ptr(), rotations.data_ptr(),
                                                  None if ctx.radii is None else ctx.radii.data_ptr(),
                                                  viewmatrix.data_ptr(), campos.data_ptr(), g.data_ptr(),
                                                  d_means.data_ptr(), d_rot.data_ptr(), _lib.current_stream_ptr()),
                       "cgx_all_map_bwd")
        return d_means, None, d_rot, None, None, None


def plane_map(means3D, scales, rotations, viewmatrix, campos, radii=None):
    """(P,5) all_map for one camera.  viewmatrix: the (4,4) row-vector world-to-view matrix of the rasterizer
    settings; campos: (3,).  radii (optional int32 (P)): rows with radius <= 0 are skipped."""
    return _PlaneMap.apply(means3D, scales, rotations, radii, viewmatrix, campos)
