"""Generate golden vectors for the spherical-harmonics colour stage by running the reference's OWN Python function
(utils/sh_utils.py eval_sh, plain torch, CPU) on a small seeded input:

    python tests/golden/make_sh_golden.py /path/to/reference [out_dir]

The reference's CUDA twin of that function (cuda_rasterizer/forward.cu:21-72) adds 0.5, clamps at zero and records
which channels were clamped; the same three steps are applied to eval_sh's result here, as the reference's Python
callers do (`torch.clamp_min(sh2rgb + 0.5, 0.0)`).  Stored: the inputs, and per degree 0..3 the colours and the
clamp flags.  tests/test_sh_golden.py pins the CPU oracle against the file on CPU and the CUDA kernel on a GPU.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main():
    ref = Path(sys.argv[1])
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    spec = importlib.util.spec_from_file_location("ref_sh_utils", ref / "utils" / "sh_utils.py")
    SH = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(SH)

    P = 1024
    gen = torch.Generator().manual_seed(160)
    means3D = (torch.rand(P, 3, generator=gen) * 2 - 1) * torch.tensor([100.0, 100.0, 15.0])
    campos = torch.tensor([3.0, -60.0, 60.0])
    # coefficients large enough that a good share of the channels is clamped at zero
    sh = torch.cat([torch.randn(P, 1, 3, generator=gen) * 1.5, torch.randn(P, 15, 3, generator=gen) * 0.3], 1)
    dirs = means3D - campos
    dirs = dirs / dirs.norm(dim=1, keepdim=True)
    out = dict(means3D=means3D.numpy(), campos=campos.numpy(), sh=sh.numpy())
    for deg in range(4):
        raw = SH.eval_sh(deg, sh.transpose(1, 2), dirs) + 0.5          # the reference wants (P, 3, coeffs)
        out[f"rgb_deg{deg}"] = torch.clamp_min(raw, 0.0).numpy()
        out[f"clamped_deg{deg}"] = (raw < 0).numpy()
        out[f"margin_deg{deg}"] = raw.abs().numpy()                    # distance from the clamp boundary
        print(deg, "clamped share", float((raw < 0).float().mean()))
    np.savez_compressed(out_dir / "sh_1024.npz", **out)
    print((out_dir / "sh_1024.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
