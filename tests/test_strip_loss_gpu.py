"""Fused strip loss (masked L1 + masked SSIM sums, forward and gradient) against the reference's formulation with
grouped convolutions (utils/loss_utils.py:27-43, 88-132), evaluated in float64 by torch and differentiated by
autograd."""
import math

import pytest
import torch
import torch.nn.functional as F

import util  # noqa: F401

pytestmark = pytest.mark.gpu


def _window(channel, dtype, device):
    g = torch.tensor([math.exp(-((x - 5) ** 2) / float(2 * 1.5 ** 2)) for x in range(11)], dtype=torch.float32)
    g = (g / g.sum()).unsqueeze(1)
    w2 = g.mm(g.t()).float().unsqueeze(0).unsqueeze(0)
    return w2.expand(channel, 1, 11, 11).contiguous().to(device=device, dtype=dtype)


def _reference_sums(img1, img2, mask):
    c = img1.shape[0]
    w = _window(c, img1.dtype, img1.device)
    m = mask.unsqueeze(0).to(img1.dtype)
    l1 = (torch.abs(img1 - img2) * m).sum()
    mu1 = F.conv2d(img1, w, padding=5, groups=c)
    mu2 = F.conv2d(img2, w, padding=5, groups=c)
    s1 = F.conv2d(img1 * img1, w, padding=5, groups=c) - mu1.pow(2)
    s2 = F.conv2d(img2 * img2, w, padding=5, groups=c) - mu2.pow(2)
    s12 = F.conv2d(img1 * img2, w, padding=5, groups=c) - mu1 * mu2
    C1, C2 = 0.01 ** 2, 0.03 ** 2
    ssim = ((2 * mu1 * mu2 + C1) * (2 * s12 + C2)) / ((mu1.pow(2) + mu2.pow(2) + C1) * (s1 + s2 + C2))
    return l1, (ssim * m).sum()


@pytest.mark.parametrize("shape,masked", [((3, 75, 200), False), ((3, 64, 48), True), ((1, 7, 9), True),
                                          ((3, 400, 1600), False)])
def test_strip_loss_matches_convolution_form(cuda_device, shape, masked):
    from cgx.strip_loss import strip_loss_sums

    gen = torch.Generator().manual_seed(sum(shape))
    img = torch.rand(shape, generator=gen)
    # a ground truth correlated with the image (as in training), plus flat regions where sigma ~ 0
    gt = (img * 0.7 + 0.3 * torch.rand(shape, generator=gen)).clamp(0, 1)
    gt[:, : shape[1] // 4] = 0.5
    mask = (torch.rand(shape[1:], generator=gen) > 0.3) if masked else torch.ones(shape[1:], dtype=torch.bool)

    x = img.to(cuda_device).requires_grad_(True)
    l1, ss = strip_loss_sums(x, gt.to(cuda_device), mask.to(cuda_device) if masked else None)
    (0.8 * l1 - 0.2 * ss).backward()

    x64 = img.double().to(cuda_device).requires_grad_(True)
    rl1, rss = _reference_sums(x64, gt.double().to(cuda_device), mask.to(cuda_device))
    (0.8 * rl1 - 0.2 * rss).backward()

    n = img.numel()
    assert abs(l1.item() - rl1.item()) <= 1e-5 * n ** 0.5 + 1e-6 * abs(rl1.item())
    assert abs(ss.item() - rss.item()) <= 1e-5 * n ** 0.5 + 1e-5 * abs(rss.item())
    ga, gb = x.grad.double(), x64.grad
    assert ((ga - gb).norm() / gb.norm()).item() <= 1e-4
    assert (ga - gb).abs().max().item() <= 1e-4 * gb.abs().max().item() + 1e-6


def test_strip_loss_refuses_cpu_tensors():
    from cgx.strip_loss import strip_loss_sums

    with pytest.raises(RuntimeError, match="CUDA"):
        strip_loss_sums(torch.zeros(3, 8, 8), torch.zeros(3, 8, 8))


def _reference_normal(depth, fx, fy, cx, cy):
    """utils/graphics_utils.py:87-152 (depth2point_cam / ndc_2_cam / depth_pcd2normal without offsets)."""
    H, W = depth.shape
    xs = torch.arange(W, dtype=depth.dtype, device=depth.device)
    ys = torch.arange(H, dtype=depth.dtype, device=depth.device)
    gx, gy = torch.meshgrid(xs, ys, indexing="xy")
    xyz = torch.stack([(gx - cx) / fx * depth, (gy - cy) / fy * depth, depth], -1)
    bottom, top = xyz[2:H, 1:W - 1], xyz[0:H - 2, 1:W - 1]
    right, left = xyz[1:H - 1, 2:W], xyz[1:H - 1, 0:W - 2]
    n = torch.cross(right - left, top - bottom, dim=-1)
    n = F.normalize(n, p=2, dim=-1)
    return F.pad(n.permute(2, 0, 1), (1, 1, 1, 1), mode="constant")


@pytest.mark.parametrize("shape", [(60, 90), (3, 3), (2, 5), (240, 320)])
def test_depth_normal_matches_tensor_form(cuda_device, shape):
    from cgx.strip_loss import depth_normal

    H, W = shape
    gen = torch.Generator().manual_seed(H * W)
    yy, xx = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
    depth = 20.0 + 0.05 * xx + 0.03 * yy + torch.rand(H, W, generator=gen)        # a tilted, rough surface
    fx, fy, cx, cy = 0.8 * W, 0.8 * W, W / 2.0, H / 2.0
    cot = torch.randn(3, H, W, generator=gen)

    d = depth.to(cuda_device).requires_grad_(True)
    n = depth_normal(d, fx, fy, cx, cy)
    (n * cot.to(cuda_device)).sum().backward()

    d64 = depth.double().to(cuda_device).requires_grad_(True)
    n64 = _reference_normal(d64, fx, fy, cx, cy)
    (n64 * cot.double().to(cuda_device)).sum().backward()

    assert n.shape == (3, H, W)
    assert (n - n64.float()).abs().max().item() <= 2e-5
    if H > 2 and W > 2:
        ga, gb = d.grad.double(), d64.grad
        assert ((ga - gb).norm() / gb.norm()).item() <= 1e-3          # float32 differences of nearby points
    else:
        assert not n.any() and not d.grad.any()
