"""Fused strip loss (masked L1 + masked SSIM sums, forward and gradient) against the reference's formulation with
grouped convolutions (utils/loss_utils.py:27-43, 88-132), evaluated in float64 by torch and differentiated by
autograd."""
import pytest
import torch

import util  # noqa: F401
from util_loss import reference_normal as _reference_normal
from util_loss import reference_sums as _reference_sums

pytestmark = pytest.mark.gpu


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
