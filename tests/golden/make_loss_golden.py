"""Generate golden vectors for the strip loss and the normal-from-depth image by running the reference's OWN Python
functions (plain torch, CPU) on small seeded inputs:

    python tests/golden/make_loss_golden.py /path/to/reference [out_dir]

  utils/loss_utils.py      pixelwise_l1_with_mask, pixelwise_ssim_with_mask     (float32, as upstream runs them)
  utils/graphics_utils.py  normal_from_depth_image (no offsets)                 (float32)

Stored per case: the inputs, the two masked sums, d(0.8*l1_sum - 0.2*ssim_sum)/d(image) from autograd, the normal
image and d(sum(normal * cotangent))/d(depth).  The files are a few tens of KB; tests/test_loss_golden.py pins the
float64 restatement used by the GPU tests against them on CPU, and the CUDA kernels against them on a GPU.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = Path(sys.argv[1])
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    LU = _load(ref / "utils" / "loss_utils.py", "ref_loss_utils")
    GU = _load(ref / "utils" / "graphics_utils.py", "ref_graphics_utils")
    for name, (C, H, W), masked in (("loss_3x40x56", (3, 40, 56), True), ("loss_3x33x17", (3, 33, 17), False)):
        gen = torch.Generator().manual_seed(C * H * W)
        img = torch.rand(C, H, W, generator=gen)
        gt = (img * 0.7 + 0.3 * torch.rand(C, H, W, generator=gen)).clamp(0, 1)
        gt[:, : H // 4] = 0.5
        mask = (torch.rand(H, W, generator=gen) > 0.3) if masked else torch.ones(H, W, dtype=torch.bool)
        x = img.clone().requires_grad_(True)
        l1 = LU.pixelwise_l1_with_mask(x, gt, mask).sum()
        ss = LU.pixelwise_ssim_with_mask(x, gt, mask).sum()
        (0.8 * l1 - 0.2 * ss).backward()

        yy, xx = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32),
                                indexing="ij")
        depth = 20.0 + 0.05 * xx + 0.03 * yy + torch.rand(H, W, generator=gen)
        fx, fy, cx, cy = 0.8 * W, 0.8 * W, W / 2.0, H / 2.0
        K = torch.tensor([[fx, 0, cx], [0, fy, cy], [0, 0, 1]]).float()
        cot = torch.randn(3, H, W, generator=gen)
        d = depth.clone().requires_grad_(True)
        normal = GU.normal_from_depth_image(d, K, torch.eye(4)).permute(2, 0, 1)
        (normal * cot).sum().backward()

        np.savez_compressed(out_dir / f"{name}.npz", img=img.numpy(), gt=gt.numpy(), mask=mask.numpy(),
                            l1_sum=np.float64(l1.item()), ssim_sum=np.float64(ss.item()), d_img=x.grad.numpy(),
                            depth=depth.numpy(), intrinsics=np.array([fx, fy, cx, cy], dtype=np.float64),
                            cot=cot.numpy(), normal=normal.detach().numpy(), d_depth=d.grad.numpy())
        print(name, float(l1), float(ss), (out_dir / f"{name}.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
