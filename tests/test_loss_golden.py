"""Golden vectors made by the reference's own Python functions (tests/golden/make_loss_golden.py): they pin the
restatement the loss tests use (CPU, float64 and float32), and the CUDA kernels (GPU)."""
import numpy as np
import pytest
import torch

import util
from util_loss import reference_normal, reference_sums

CASES = ["loss_3x40x56", "loss_3x33x17"]


def _load(name):
    z = np.load(util.GOLDEN / f"{name}.npz")
    return {k: (torch.from_numpy(z[k]) if z[k].ndim else float(z[k])) for k in z.files}


@pytest.mark.parametrize("name", CASES)
def test_restatement_matches_reference_functions(name):
    g = _load(name)
    for dtype, tol in ((torch.float64, 2e-5), (torch.float32, 2e-5)):
        x = g["img"].to(dtype).requires_grad_(True)
        l1, ss = reference_sums(x, g["gt"].to(dtype), g["mask"])
        (0.8 * l1 - 0.2 * ss).backward()
        assert abs(l1.item() - g["l1_sum"]) <= 1e-6 * abs(g["l1_sum"]) + 1e-4
        assert abs(ss.item() - g["ssim_sum"]) <= 1e-6 * abs(g["ssim_sum"]) + 1e-3
        assert util.rel_l2(x.grad.float(), g["d_img"]) <= tol
        fx, fy, cx, cy = g["intrinsics"].tolist()
        d = g["depth"].to(dtype).requires_grad_(True)
        n = reference_normal(d, fx, fy, cx, cy)
        (n * g["cot"].to(dtype)).sum().backward()
        assert (n.float() - g["normal"]).abs().max().item() <= 2e-5
        assert util.rel_l2(d.grad.float(), g["d_depth"]) <= 1e-3      # float32 goldens: differences of nearby points


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernels_match_reference_functions(name, cuda_device):
    from cgx.strip_loss import depth_normal, strip_loss_sums

    g = _load(name)
    dev = cuda_device
    x = g["img"].to(dev).requires_grad_(True)
    masked = not bool(g["mask"].all())
    l1, ss = strip_loss_sums(x, g["gt"].to(dev), g["mask"].to(dev) if masked else None)
    (0.8 * l1 - 0.2 * ss).backward()
    assert abs(l1.item() - g["l1_sum"]) <= 1e-5 * abs(g["l1_sum"])
    assert abs(ss.item() - g["ssim_sum"]) <= 1e-5 * abs(g["ssim_sum"])
    assert util.rel_l2(x.grad.cpu(), g["d_img"]) <= 1e-4
    fx, fy, cx, cy = g["intrinsics"].tolist()
    d = g["depth"].to(dev).requires_grad_(True)
    n = depth_normal(d, fx, fy, cx, cy)
    (n * g["cot"].to(dev)).sum().backward()
    assert (n.cpu() - g["normal"]).abs().max().item() <= 2e-5
    assert util.rel_l2(d.grad.cpu(), g["d_depth"]) <= 2e-3            # both sides float32
