"""Float64-capable restatements of the reference's loss-side tensor code, shared by the loss tests.  They are
pinned against outputs of the reference's own functions in tests/test_loss_golden.py."""
import math

import torch
import torch.nn.functional as F


def window(channel, dtype, device):
    g = torch.tensor([math.exp(-((x - 5) ** 2) / float(2 * 1.5 ** 2)) for x in range(11)], dtype=torch.float32)
    g = (g / g.sum()).unsqueeze(1)
    w2 = g.mm(g.t()).float().unsqueeze(0).unsqueeze(0)
    return w2.expand(channel, 1, 11, 11).contiguous().to(device=device, dtype=dtype)


def reference_sums(img1, img2, mask):
    c = img1.shape[0]
    w = window(c, img1.dtype, img1.device)
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


def reference_normal(depth, fx, fy, cx, cy):
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
