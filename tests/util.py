"""Shared helpers for the parity tests."""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "citygs-x_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

from cgx import synthetic as S  # noqa: E402

GOLDEN = Path(__file__).resolve().parent / "golden"


def make_case(cfg=1, n=20000, res=(320, 180), cam_idx=0, seed_offset=0, big_scales=False):
    """Gaussians + one camera of benchmark configuration `cfg`, shrunk to (n, res)."""
    g, cams = S.config(cfg, n_gaussians=n, res=res)
    cam = cams[cam_idx]
    if big_scales:   # a few very large splats: many tiles per Gaussian, long per-tile lists
        gen = torch.Generator().manual_seed(7 + seed_offset)
        idx = torch.randperm(n, generator=gen)[: max(1, n // 50)]
        g["scales"][idx] *= 40.0
    g["rgb"] = S.colours_for(g, cam)
    g["all_map"] = S.build_all_map(g["means3D"], g["scales"], g["rotations"], cam)
    return g, cam


def cotangents(cam, seed=0):
    gen = torch.Generator().manual_seed(1234 + seed)
    return dict(color=torch.randn(3, cam.H, cam.W, generator=gen),
                all_map=torch.randn(5, cam.H, cam.W, generator=gen),
                plane_depth=torch.randn(1, cam.H, cam.W, generator=gen))


def cam_dict(cam, bg=None):
    return dict(W=cam.W, H=cam.H, tanfovx=cam.tanfovx, tanfovy=cam.tanfovy, viewmatrix=cam.viewmatrix,
                projmatrix=cam.projmatrix, bg=torch.zeros(3) if bg is None else bg)


def settings_for(cam, device, bg=None, render_geo=True, debug=False):
    from diff_gaussian_rasterization import GaussianRasterizationSettings

    return GaussianRasterizationSettings(
        image_height=cam.H, image_width=cam.W, tanfovx=cam.tanfovx, tanfovy=cam.tanfovy,
        bg=(torch.zeros(3) if bg is None else bg).to(device), scale_modifier=1.0,
        viewmatrix=cam.viewmatrix.to(device), projmatrix=cam.projmatrix.to(device), sh_degree=3,
        campos=cam.campos.to(device), prefiltered=False, render_geo=render_geo, debug=debug)


def cuda_args(stats=None):
    return {"mode": "train", "world_size": "1", "global_rank": "0", "local_rank": "0", "mp_world_size": "1",
            "mp_rank": "0", "log_folder": "/tmp", "log_interval": "10", "iteration": "2", "zhx_debug": "False",
            "zhx_time": "False", "dist_global_strategy": "", "avoid_pixel_all2all": False,
            "stats_collector": {} if stats is None else stats}


def rel_l2(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    d = (a - b).norm()
    n = b.norm()
    return float(d / n) if n > 0 else float(d)


def decode_binning(buf, R):
    """point_list / sorted keys out of a binning scratch buffer (reference layout: four 128-byte aligned arrays)."""
    from diff_gaussian_rasterization import _C

    class L(_C._Carver):
        pass

    lay = (L().add("point_list", torch.int32, R).add("point_list_unsorted", torch.int32, R)
           .add("point_list_keys", torch.int64, R).add("point_list_keys_unsorted", torch.int64, R))
    return lay.views(buf)


def decode_image(buf, N, n_ranges):
    from diff_gaussian_rasterization import _C

    lay = (_C._Carver().add("accum_alpha", torch.float32, N).add("n_contrib", torch.int32, N)
           .add("n_contrib2loss", torch.int32, N).add("ranges", torch.int32, 2 * n_ranges))
    return lay.views(buf)
