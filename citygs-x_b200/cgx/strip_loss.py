"""Loss on a rendered strip: masked L1 and masked 11x11 Gaussian-window SSIM against the ground-truth strip, as the
reference computes them on every rank's local rows (utils/loss_utils.py:88-132 `pixelwise_l1_with_mask`,
`pixelwise_ssim_with_mask`; gaussian_renderer/loss_distribution.py:2835-2885 sums them and divides by the number of
pixels of the whole image times 3).  The reference runs five grouped 11x11 convolutions and a dozen element-wise
kernels forward, and autograd's transposed convolutions backward; here the forward is one kernel and the backward
is one kernel (`cgx_strip_loss_fwd` / `cgx_strip_loss_bwd`).

    l1_sum, ssim_sum = strip_loss_sums(image, gt, mask)        # device scalars, differentiable towards `image`
    Ll1, ssim_loss = l1_sum / (n_pixels * 3), ssim_sum / (n_pixels * 3)
"""
from __future__ import annotations

import torch

from diff_gaussian_rasterization import _lib


class _StripLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, image, gt, mask):
        if not image.is_cuda or image.dtype != torch.float32 or not gt.is_cuda or gt.dtype != torch.float32:
            raise RuntimeError("strip_loss: image and gt must be float32 CUDA tensors (no CPU path)")
        if image.ndim != 3 or gt.shape != image.shape:
            raise RuntimeError("strip_loss: image and gt must both be (C, H, W)")
        image, gt = image.contiguous(), gt.contiguous()
        C, H, W = image.shape
        if mask is not None:
            if mask.shape != (H, W) or not mask.is_cuda:
                raise RuntimeError("strip_loss: mask must be a (H, W) CUDA tensor")
            mask = mask.to(torch.bool).contiguous()
        sums = torch.empty(2, device=image.device, dtype=torch.float64)
        need = image.requires_grad
        maps = torch.empty(3, C, H, W, device=image.device) if need else None
        if C * H * W:
            with torch.cuda.device(image.device):
                _lib.check(_lib.lib().cgx_strip_loss_fwd(
                    C, H, W, image.data_ptr(), gt.data_ptr(), None if mask is None else mask.data_ptr(),
                    sums.data_ptr(), *([maps[i].data_ptr() for i in range(3)] if need else [None, None, None]),
                    _lib.current_stream_ptr()), "cgx_strip_loss_fwd")
        else:
            sums.zero_()
        ctx.save_for_backward(image, gt, mask, maps)
        sums = sums.to(torch.float32)
        return sums[0], sums[1]

    @staticmethod
    def backward(ctx, g_l1, g_ssim):
        image, gt, mask, maps = ctx.saved_tensors
        C, H, W = image.shape
        zero = torch.zeros((), device=image.device)
        weights = torch.stack([g_l1 if g_l1 is not None else zero, g_ssim if g_ssim is not None else zero]) \
            .to(torch.float32).contiguous()
        grad = torch.empty_like(image)
        if C * H * W:
            with torch.cuda.device(image.device):
                _lib.check(_lib.lib().cgx_strip_loss_bwd(
                    C, H, W, image.data_ptr(), gt.data_ptr(), None if mask is None else mask.data_ptr(),
                    weights.data_ptr(), maps[0].data_ptr(), maps[1].data_ptr(), maps[2].data_ptr(), grad.data_ptr(),
                    _lib.current_stream_ptr()), "cgx_strip_loss_bwd")
        return grad, None, None


def strip_loss_sums(image, gt, mask=None):
    """(sum of mask * |image - gt|, sum of mask * SSIM map) over a (C, H, W) strip; `mask` (H, W) bool or None."""
    return _StripLoss.apply(image, gt, mask)


class _DepthNormal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, depth, fx, fy, cx, cy):
        if not depth.is_cuda or depth.dtype != torch.float32 or depth.ndim != 2:
            raise RuntimeError("depth_normal: depth must be a (H, W) float32 CUDA tensor (no CPU path)")
        depth = depth.contiguous()
        H, W = depth.shape
        normal = torch.empty(3, H, W, device=depth.device)
        if H * W:
            with torch.cuda.device(depth.device):
                _lib.check(_lib.lib().cgx_depth_normal_fwd(H, W, fx, fy, cx, cy, depth.data_ptr(), normal.data_ptr(),
                                                           _lib.current_stream_ptr()), "cgx_depth_normal_fwd")
        ctx.save_for_backward(depth)
        ctx.k = (fx, fy, cx, cy)
        return normal

    @staticmethod
    def backward(ctx, g):
        (depth,) = ctx.saved_tensors
        H, W = depth.shape
        out = torch.empty_like(depth)
        if H * W:
            g = g.contiguous()
            with torch.cuda.device(depth.device):
                _lib.check(_lib.lib().cgx_depth_normal_bwd(H, W, *ctx.k, depth.data_ptr(), g.data_ptr(),
                                                           out.data_ptr(), _lib.current_stream_ptr()),
                           "cgx_depth_normal_bwd")
        return out, None, None, None, None


def depth_normal(depth, fx, fy, cx, cy):
    """(3, H, W) camera-space normals of a (H, W) depth image: the reference's ``render_normal`` at scale 1 without
    offsets (gaussian_renderer/__init__.py:1311-1323; utils/graphics_utils.py:87-152), differentiable towards the
    depth (this is where the plane-depth cotangent of the rasterizer comes from in training)."""
    return _DepthNormal.apply(depth, float(fx), float(fy), float(cx), float(cy))
