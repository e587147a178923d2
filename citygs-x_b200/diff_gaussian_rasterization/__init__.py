"""Drop-in replacement for CityGS-X's ``diff_gaussian_rasterization`` package on B200 (sm_100a).

Public surface, argument order, output tuples and gradient contract follow the reference package
(RAST/diff_gaussian_rasterization/__init__.py): ``GaussianRasterizationSettings`` (:314-327),
``GaussianRasterizer`` with ``markVisible`` / ``preprocess_gaussians`` / ``visible_filter`` /
``render_gaussians`` (:329-405), the module-level ``preprocess_gaussians`` / ``render_gaussians`` (:27-44,
:155-180), ``load_image_tiles_by_pos`` / ``merge_image_tiles_by_pos`` (:509-537) and the raw ``_C`` module.
The two-stage split (per-Gaussian preprocess, then per-tile render, with the caller's all-to-all in between)
is the reference's.  All compute runs in hand-written CUDA kernels behind the C ABI of
``include/cgx_raster.h``; this file is autograd plumbing only.
"""
from typing import NamedTuple

import torch
import torch.nn as nn

from . import _C  # noqa: F401  (callers reach into diff_gaussian_rasterization._C directly)


def cpu_deep_copy_tuple(input_tuple):
    return tuple(item.cpu().clone() if isinstance(item, torch.Tensor) else item for item in input_tuple)


# ----------------------------------------------------------------------------- preprocess
def preprocess_gaussians(means3D, scales, rotations, sh, opacities, raster_settings, cuda_args):
    return _PreprocessGaussians.apply(means3D, scales, rotations, sh, opacities, raster_settings, cuda_args)


class _PreprocessGaussians(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means3D, scales, rotations, sh, opacities, raster_settings, cuda_args):
        rs = raster_settings
        num_rendered, means2D, depths, radii, cov3D, conic_opacity, rgb, clamped = _C.preprocess_gaussians(
            means3D, scales, rotations, sh, opacities, rs.scale_modifier, rs.viewmatrix, rs.projmatrix,
            rs.tanfovx, rs.tanfovy, rs.image_height, rs.image_width, rs.sh_degree, rs.campos, rs.prefiltered,
            rs.debug, cuda_args)
        ctx.raster_settings = rs
        ctx.cuda_args = cuda_args
        ctx.num_rendered = num_rendered
        # cov3D is recomputed in the backward kernel; it is still returned by _C for drop-in parity
        ctx.save_for_backward(means3D, scales, rotations, sh, radii)
        ctx.mark_non_differentiable(radii, depths)
        return means2D, rgb, conic_opacity, radii, depths

    @staticmethod
    def backward(ctx, grad_means2D, grad_rgb, grad_conic_opacity, grad_radii, grad_depths):
        rs = ctx.raster_settings
        means3D, scales, rotations, sh, radii = ctx.saved_tensors
        P = means3D.shape[0]
        if grad_means2D is None:
            grad_means2D = torch.zeros(P, 2, dtype=means3D.dtype, device=means3D.device)
        if grad_conic_opacity is None:
            grad_conic_opacity = torch.zeros(P, 4, dtype=means3D.dtype, device=means3D.device)
        dL_dmeans3D, dL_dscales, dL_drotations, dL_dsh, dL_dopacity = _C.preprocess_gaussians_backward(
            radii, None, None, means3D, scales, rotations, sh, rs.scale_modifier, rs.viewmatrix, rs.projmatrix,
            rs.tanfovx, rs.tanfovy, rs.image_height, rs.image_width, rs.sh_degree, rs.campos, grad_means2D,
            grad_conic_opacity, grad_rgb, ctx.num_rendered, rs.debug, ctx.cuda_args)
        return dL_dmeans3D, dL_dscales, dL_drotations, dL_dsh, dL_dopacity, None, None


# ----------------------------------------------------------------------------- render
def render_gaussians(means2D, means2D_abs, conic_opacity, rgb, all_map, depths, radii, compute_locally,
                     extended_compute_locally, raster_settings, cuda_args):
    return _RenderGaussians.apply(means2D, means2D_abs, conic_opacity, rgb, all_map, depths, radii, compute_locally,
                                  extended_compute_locally, raster_settings, cuda_args)


class _RenderGaussians(torch.autograd.Function):
    @staticmethod
    def forward(ctx, means2D, means2D_abs, conic_opacity, rgb, all_maps, depths, radii, compute_locally,
                extended_compute_locally, raster_settings, cuda_args):
        rs = raster_settings
        local = extended_compute_locally if cuda_args["avoid_pixel_all2all"] else compute_locally
        (num_rendered, color, n_render, n_consider, n_contrib, out_observe, out_all_map, out_plane_depth,
         geomBuffer, binningBuffer, imgBuffer) = _C.render_gaussians(
            rs.bg, rs.image_height, rs.image_width, means2D, depths, radii, conic_opacity, rgb, local,
            rs.viewmatrix, rs.campos, rs.tanfovx, rs.tanfovy, all_maps, rs.render_geo, rs.debug, cuda_args)
        ctx.raster_settings = rs
        ctx.cuda_args = cuda_args
        ctx.num_rendered = num_rendered
        ctx.save_for_backward(means2D, conic_opacity, rgb, all_maps, out_all_map, geomBuffer, binningBuffer,
                              imgBuffer, compute_locally)
        ctx.mark_non_differentiable(n_render, n_consider, n_contrib, out_observe)
        return color, n_render, n_consider, n_contrib, out_observe, out_all_map, out_plane_depth

    @staticmethod
    def backward(ctx, grad_color, grad_n_render, grad_n_consider, grad_n_contrib, grad_out_observe,
                 grad_out_all_map, grad_out_plane_depth):
        rs = ctx.raster_settings
        (means2D, conic_opacity, rgb, all_maps, all_map_pixels, geomBuffer, binningBuffer, imgBuffer,
         compute_locally) = ctx.saved_tensors
        H, W = rs.image_height, rs.image_width
        if grad_color is None:
            grad_color = torch.zeros(3, H, W, dtype=means2D.dtype, device=means2D.device)
        if grad_out_all_map is None:
            grad_out_all_map = torch.zeros(5, H, W, dtype=means2D.dtype, device=means2D.device)
        if grad_out_plane_depth is None:
            grad_out_plane_depth = torch.zeros(1, H, W, dtype=means2D.dtype, device=means2D.device)
        dL_dmeans2D, dL_dmeans2D_abs, dL_dconic_opacity, dL_dcolors, dL_dall_map = _C.render_gaussians_backward_2d(
            rs.bg, rs.tanfovx, rs.tanfovy, all_map_pixels, all_maps, ctx.num_rendered, geomBuffer, binningBuffer,
            imgBuffer, compute_locally, grad_color, grad_out_all_map, grad_out_plane_depth, means2D, conic_opacity,
            rgb, rs.render_geo, rs.debug, ctx.cuda_args)
        return (dL_dmeans2D, dL_dmeans2D_abs, dL_dconic_opacity, dL_dcolors, dL_dall_map,
                None, None, None, None, None, None)


# ----------------------------------------------------------------------------- settings / module
class GaussianRasterizationSettings(NamedTuple):
    image_height: int
    image_width: int
    tanfovx: float
    tanfovy: float
    bg: torch.Tensor
    scale_modifier: float
    viewmatrix: torch.Tensor
    projmatrix: torch.Tensor
    sh_degree: int
    campos: torch.Tensor
    prefiltered: bool
    render_geo: bool
    debug: bool


class GaussianRasterizer(nn.Module):
    def __init__(self, raster_settings):
        super().__init__()
        self.raster_settings = raster_settings

    def markVisible(self, positions):
        with torch.no_grad():
            rs = self.raster_settings
            return _C.mark_visible(positions, rs.viewmatrix, rs.projmatrix)

    def preprocess_gaussians(self, means3D, scales, rotations, shs, opacities, cuda_args=None):
        return preprocess_gaussians(means3D, scales, rotations, shs, opacities, self.raster_settings, cuda_args)

    def visible_filter(self, means3D, scales=None, rotations=None, cov3D_precomp=None):
        rs = self.raster_settings
        if scales is None:
            scales = torch.Tensor([])
        if rotations is None:
            rotations = torch.Tensor([])
        if cov3D_precomp is None:
            cov3D_precomp = torch.Tensor([])
        with torch.no_grad():
            return _C.rasterize_aussians_filter(means3D, scales, rotations, rs.scale_modifier, cov3D_precomp,
                                                rs.viewmatrix, rs.projmatrix, rs.tanfovx, rs.tanfovy,
                                                rs.image_height, rs.image_width, rs.prefiltered, rs.debug)

    def render_gaussians(self, means2D, means2D_abs, conic_opacity, rgb, all_map, depths, radii, compute_locally,
                         extended_compute_locally, cuda_args=None):
        return render_gaussians(means2D, means2D_abs, conic_opacity, rgb, all_map, depths, radii, compute_locally,
                                extended_compute_locally, self.raster_settings, cuda_args)


# ----------------------------------------------------------------------------- image-tile helpers (legacy API)
class _LoadImageTilesByPos(torch.autograd.Function):
    @staticmethod
    def forward(ctx, local_image_rect, all_tiles_pos, image_height, image_width, touched_pixels_rect,
                touched_tiles_rect):
        ctx.save_for_backward(all_tiles_pos)
        ctx.args = (image_height, image_width, touched_pixels_rect)
        y0, y1, x0, x1 = touched_pixels_rect
        return _C.load_image_tiles_by_pos(local_image_rect, all_tiles_pos, image_height, image_width, y0, x0,
                                          y1 - y0, x1 - x0)

    @staticmethod
    def backward(ctx, grad_image_tiles):
        (all_tiles_pos,) = ctx.saved_tensors
        image_height, image_width, (y0, y1, x0, x1) = ctx.args
        g = _C.set_image_tiles_by_pos(all_tiles_pos, grad_image_tiles, image_height, image_width, y0, x0,
                                      y1 - y0, x1 - x0)
        return g, None, None, None, None, None


class _MergeImageTilesByPos(torch.autograd.Function):
    @staticmethod
    def forward(ctx, all_tiles_pos, image_tiles, image_height, image_width, touched_pixels_rect,
                touched_tiles_rect):
        ctx.save_for_backward(all_tiles_pos)
        ctx.args = (image_height, image_width, touched_pixels_rect)
        y0, y1, x0, x1 = touched_pixels_rect
        return _C.set_image_tiles_by_pos(all_tiles_pos, image_tiles, image_height, image_width, y0, x0,
                                         y1 - y0, x1 - x0)

    @staticmethod
    def backward(ctx, grad_rect):
        (all_tiles_pos,) = ctx.saved_tensors
        image_height, image_width, (y0, y1, x0, x1) = ctx.args
        g = _C.load_image_tiles_by_pos(grad_rect, all_tiles_pos, image_height, image_width, y0, x0, y1 - y0, x1 - x0)
        return None, g, None, None, None, None


def load_image_tiles_by_pos(local_image_rect, all_tiles_pos, image_height, image_width, touched_pixels_rect,
                            touched_tiles_rect):
    return _LoadImageTilesByPos.apply(local_image_rect, all_tiles_pos, image_height, image_width,
                                      touched_pixels_rect, touched_tiles_rect)


def merge_image_tiles_by_pos(all_tiles_pos, image_tiles, image_height, image_width, touched_pixels_rect,
                             touched_tiles_rect):
    return _MergeImageTilesByPos.apply(all_tiles_pos, image_tiles, image_height, image_width, touched_pixels_rect,
                                       touched_tiles_rect)
