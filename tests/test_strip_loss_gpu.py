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
