"""Spherical-harmonics colour stage against golden vectors made by the reference's own Python function
(utils/sh_utils.py eval_sh, run by tests/golden/make_sh_golden.py): the CPU oracle on CPU, the CUDA kernel on a GPU."""
import numpy as np
import pytest
import torch

import util

TOL = 1e-5          # colours are sums of at most 16 products of O(1) numbers in float32
EDGE = 1e-5         # a channel this close to the clamp boundary may fall on either side


def _golden():
    z = np.load(util.GOLDEN / "sh_1024.npz")
    return {k: torch.from_numpy(z[k]) for k in z.files}


def _check(rgb, clamped, g, deg):
    assert (rgb - g[f"rgb_deg{deg}"]).abs().max().item() <= TOL
    decided = g[f"margin_deg{deg}"] > EDGE
    assert torch.equal(clamped[decided], g[f"clamped_deg{deg}"][decided])
    assert bool(g[f"clamped_deg{deg}"].any()) and not bool(g[f"clamped_deg{deg}"].all())


@pytest.mark.parametrize("deg", [0, 1, 2, 3])
def test_oracle_sh_matches_reference_function(deg):
    from oracle import cpu_raster as O

    g = _golden()
    rgb, clamped = O.sh_to_rgb(g["means3D"], g["campos"], g["sh"], deg)
    _check(rgb, clamped, g, deg)


@pytest.mark.gpu
@pytest.mark.parametrize("deg", [0, 1, 2, 3])
def test_kernel_sh_matches_reference_function(deg, cuda_device):
    from diff_gaussian_rasterization import _lib

    g = _golden()
    dev = cuda_device
    P = g["means3D"].shape[0]
    rgb = torch.empty(P, 3, device=dev)
    clamped = torch.empty(P, 3, dtype=torch.bool, device=dev)
    m, sh, cp = g["means3D"].to(dev), g["sh"].to(dev), g["campos"].to(dev)
    st = _lib.lib().cgx_sh_to_rgb(P, deg, 16, m.data_ptr(), cp.data_ptr(), sh.data_ptr(), rgb.data_ptr(),
                                  clamped.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    _check(rgb.cpu(), clamped.cpu(), g, deg)
