"""torch-on-CPU oracle of the CityGS-X rasterizer hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  Only ``tests/``, the
smoke check and the benchmark's CPU-baseline legs may use it, and only as the
checker / the thing timed *as the CPU baseline* — never as a fallback.

The functions take and return CPU ``torch`` tensors with the shapes and dtypes
of the reference's operator API (RAST/diff_gaussian_rasterization/__init__.py,
RAST/rasterize_points.cu); the arithmetic lives in ``cgx_oracle.c`` (sequential
C restatement of each reference kernel, OpenMP over Gaussians / tiles), loaded
with ctypes.  ``preprocess_gaussians`` / ``render_gaussians`` mirror the
reference's two autograd stages, forward and backward, so that the parity
tests read like calls of the reference API.

Parity status: the reference has no tests or golden vectors for this path; the
oracle is pinned by outputs of the reference's own CUDA extension captured on a
B200 (tests/golden/*.npz, produced by tests/golden/make_golden.py).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
_SRC = HERE / "cgx_oracle.c"
_SO = HERE / "libcgx_oracle.so"
_lib = None

BLOCK_X = 16
BLOCK_Y = 16


def build(force: bool = False) -> Path:
    if force or not _SO.exists() or _SO.stat().st_mtime < _SRC.stat().st_mtime:
        cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
               str(_SRC), "-o", str(_SO), "-lm"]
        subprocess.run(cmd, check=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(_SO))
        _lib.orc_tile_count.restype = C.c_int64
        _lib.orc_higher_msb.restype = C.c_uint32
    return _lib


def _p(t: torch.Tensor | None):
    if t is None:
        return C.c_void_p(0)
    assert t.device.type == "cpu" and t.is_contiguous(), "oracle takes contiguous CPU tensors"
    return C.c_void_p(t.data_ptr())


def _f(t, shape=None):
    t = t.detach().to(torch.float32).contiguous()
    return t


def tile_grid(W: int, H: int):
    return (W + BLOCK_X - 1) // BLOCK_X, (H + BLOCK_Y - 1) // BLOCK_Y


def higher_msb(n: int) -> int:
    return int(lib().orc_higher_msb(C.c_uint32(n)))


# ----------------------------------------------------------------------------- stage functions
def preprocess_fwd(means3D, scales, rotations, opacities, viewmatrix, projmatrix, W, H, tanfovx, tanfovy,
                   scale_modifier=1.0, want_fragile=False):
    P = means3D.shape[0]
    means3D, scales, rotations, opacities = map(_f, (means3D, scales, rotations, opacities))
    V, Pm = _f(viewmatrix), _f(projmatrix)
    means2D = torch.zeros(P, 2)
    depths = torch.zeros(P)
    radii = torch.zeros(P, dtype=torch.int32)
    cov3D = torch.zeros(P, 6)
    conic_opacity = torch.zeros(P, 4)
    fragile = torch.zeros(P, dtype=torch.uint8) if want_fragile else None
    if P:
        lib().orc_preprocess_fwd(P, _p(means3D), _p(scales), C.c_float(scale_modifier), _p(rotations), _p(opacities),
                                 _p(V), _p(Pm), W, H, C.c_float(tanfovx), C.c_float(tanfovy),
                                 _p(means2D), _p(depths), _p(radii), _p(cov3D), _p(conic_opacity), _p(fragile))
    out = (means2D, depths, radii, cov3D, conic_opacity)
    return out + (fragile.bool(),) if want_fragile else out


def filter_preprocess(means3D, scales, rotations, viewmatrix, projmatrix, W, H, tanfovx, tanfovy, scale_modifier=1.0):
    P = means3D.shape[0]
    radii = torch.zeros(P, dtype=torch.int32)
    if P:
        lib().orc_filter_preprocess(P, _p(_f(means3D)), _p(_f(scales)), C.c_float(scale_modifier), _p(_f(rotations)),
                                    _p(_f(viewmatrix)), _p(_f(projmatrix)), W, H, C.c_float(tanfovx),
                                    C.c_float(tanfovy), _p(radii))
    return radii


def mark_visible(means3D, viewmatrix):
    P = means3D.shape[0]
    out = torch.zeros(P, dtype=torch.uint8)
    if P:
        lib().orc_mark_visible(P, _p(_f(means3D)), _p(_f(viewmatrix)), _p(out))
    return out.bool()


def local2j_mask(means2D, radii, tile_bounds, W, H, avoid_pixel_all2all=False):
    """tile_bounds: int32 (ws+1) linear tile ids = division_pos * TILE_X."""
    P = means2D.shape[0]
    ws = tile_bounds.numel() - 1
    mask = torch.zeros(P, ws, dtype=torch.uint8)
    if P:
        lib().orc_local2j_mask(P, H, W, ws, _p(_f(means2D)), _p(radii.to(torch.int32).contiguous()),
                               _p(tile_bounds.to(torch.int32).contiguous()), int(avoid_pixel_all2all), _p(mask))
    return mask.bool()


def bin_and_sort(means2D, depths, radii, compute_locally, W, H):
    """updateTileTouched + scan + duplicateWithKeys + stable sort + identifyTileRanges."""
    P = means2D.shape[0]
    gx, gy = tile_grid(W, H)
    local = compute_locally.reshape(-1).to(torch.uint8).contiguous()
    means2D, depths = _f(means2D), _f(depths)
    radii = radii.to(torch.int32).contiguous()
    touched = torch.zeros(P, dtype=torch.int32)
    offsets = torch.zeros(P, dtype=torch.int32)
    R = int(lib().orc_tile_count(P, W, H, _p(radii), _p(means2D), _p(local), _p(touched), _p(offsets))) if P else 0
    keys_u = torch.zeros(R, dtype=torch.int64)
    vals_u = torch.zeros(R, dtype=torch.int32)
    keys = torch.zeros(R, dtype=torch.int64)
    vals = torch.zeros(R, dtype=torch.int32)
    ranges = torch.zeros(gx * gy, 2, dtype=torch.int32)
    if R:
        lib().orc_emit_keys(P, W, H, _p(radii), _p(means2D), _p(depths), _p(offsets), _p(local), _p(keys_u), _p(vals_u))
        bit = higher_msb(gx * gy)
        lib().orc_sort_pairs(C.c_int64(R), 32 + bit, _p(keys_u), _p(vals_u), _p(keys), _p(vals))
    lib().orc_tile_ranges(C.c_int64(R), gx * gy, _p(keys), _p(ranges))
    return dict(R=R, tiles_touched=touched, offsets=offsets, keys_unsorted=keys_u, vals_unsorted=vals_u,
                keys=keys, point_list=vals, ranges=ranges)


def render_fwd(means2D, conic_opacity, rgb, all_map, ranges, point_list, compute_locally, bg, W, H,
               tanfovx, tanfovy, render_geo=True):
    P = means2D.shape[0]
    gx, gy = tile_grid(W, H)
    local = compute_locally.reshape(-1).to(torch.uint8).contiguous()
    final_T = torch.zeros(H * W)
    n_contrib = torch.zeros(H * W, dtype=torch.int32)
    n_c2l = torch.zeros(H * W, dtype=torch.int32)
    color = torch.zeros(3, H, W)
    observe = torch.zeros(P, dtype=torch.int32)
    out_all_map = torch.zeros(5, H, W)
    plane_depth = torch.zeros(1, H, W)
    lib().orc_render_fwd(W, H, C.c_float(tanfovx), C.c_float(tanfovy), _p(ranges.contiguous()),
                         _p(point_list.contiguous()), _p(_f(means2D)), _p(_f(rgb)), _p(_f(all_map)),
                         _p(_f(conic_opacity)), _p(local), _p(_f(bg)), int(render_geo),
                         _p(final_T), _p(n_contrib), _p(n_c2l), _p(color), _p(observe), _p(out_all_map),
                         _p(plane_depth))
    n_render = torch.zeros(gx * gy, dtype=torch.int32)
    n_consider = torch.zeros(gx * gy, dtype=torch.int32)
    n_contrib_t = torch.zeros(gx * gy, dtype=torch.int32)
    lib().orc_tile_stats(W, H, _p(ranges.contiguous()), _p(n_contrib), _p(n_c2l), _p(local), _p(n_render),
                         _p(n_consider), _p(n_contrib_t))
    return dict(color=color, out_all_map=out_all_map, out_plane_depth=plane_depth, out_observe=observe,
                final_T=final_T, n_contrib_px=n_contrib, n_contrib2loss_px=n_c2l,
                n_render=n_render, n_consider=n_consider, n_contrib=n_contrib_t)


def render_bwd(means2D, conic_opacity, rgb, all_map, all_map_pixels, final_T, n_contrib_px, ranges, point_list,
               compute_locally, bg, W, H, tanfovx, tanfovy, dL_dcolor, dL_dall_map_px, dL_dplane_depth,
               render_geo=True):
    P = means2D.shape[0]
    local = compute_locally.reshape(-1).to(torch.uint8).contiguous()
    d_m2 = torch.zeros(P, 3)
    d_m2abs = torch.zeros(P, 3)
    d_conic = torch.zeros(P, 4)
    d_op = torch.zeros(P)
    d_col = torch.zeros(P, 3)
    d_map = torch.zeros(P, 5)
    lib().orc_render_bwd(P, W, H, C.c_float(tanfovx), C.c_float(tanfovy), _p(ranges.contiguous()),
                         _p(point_list.contiguous()), _p(_f(bg)), _p(_f(means2D)), _p(_f(conic_opacity)),
                         _p(_f(rgb)), _p(_f(all_map)), _p(_f(all_map_pixels)), _p(_f(final_T)),
                         _p(n_contrib_px.contiguous()), _p(local), _p(_f(dL_dcolor)), _p(_f(dL_dall_map_px)),
                         _p(_f(dL_dplane_depth)), int(render_geo),
                         _p(d_m2), _p(d_m2abs), _p(d_conic), _p(d_op), _p(d_col), _p(d_map))
    # (P,2,2)+(P,1) -> (P,4) repack of RAST/rasterize_points.cu:428-436
    d_conic_opacity = torch.stack([d_conic[:, 0], d_conic[:, 1], d_conic[:, 3], d_op], dim=1).contiguous()
    return dict(dL_dmeans2D=d_m2[:, :2].contiguous(), dL_dmeans2D_abs=d_m2abs, dL_dconic_opacity=d_conic_opacity,
                dL_drgb=d_col, dL_dall_map=d_map)


def preprocess_bwd(means3D, scales, rotations, radii, cov3D, viewmatrix, projmatrix, W, H, tanfovx, tanfovy,
                   dL_dmeans2D, dL_dconic_opacity, scale_modifier=1.0):
    P = means3D.shape[0]
    d_means = torch.zeros(P, 3)
    d_scales = torch.zeros(P, 3)
    d_rot = torch.zeros(P, 4)
    d_op = torch.zeros(P, 1)
    if P:
        lib().orc_preprocess_bwd(P, _p(_f(means3D)), _p(_f(scales)), C.c_float(scale_modifier), _p(_f(rotations)),
                                 _p(radii.to(torch.int32).contiguous()), _p(_f(cov3D)), _p(_f(viewmatrix)),
                                 _p(_f(projmatrix)), W, H, C.c_float(tanfovx), C.c_float(tanfovy),
                                 _p(_f(dL_dmeans2D)), _p(_f(dL_dconic_opacity)),
                                 _p(d_means), _p(d_scales), _p(d_rot), _p(d_op))
    return dict(dL_dmeans3D=d_means, dL_dscales=d_scales, dL_drotations=d_rot, dL_dopacity=d_op,
                dL_dsh=torch.zeros(P, 3))


def sh_to_rgb(means3D, campos, sh, degree):
    P, M = sh.shape[0], sh.shape[1]
    rgb = torch.zeros(P, 3)
    clamped = torch.zeros(P, 3, dtype=torch.uint8)
    if P:
        lib().orc_sh_to_rgb(P, degree, M, _p(_f(means3D)), _p(_f(campos)), _p(_f(sh)), _p(rgb), _p(clamped))
    return rgb, clamped.bool()


# ----------------------------------------------------------------------------- whole-path convenience
def full_step(g, cam, compute_locally=None, cot=None, render_geo=True):
    """preprocess -> bin/sort -> render -> (optional) backward, for one camera on CPU.

    ``g``: dict with means3D, scales, rotations, opacities, rgb, all_map;
    ``cam``: dict with W, H, tanfovx, tanfovy, viewmatrix, projmatrix, bg.
    ``cot``: optional dict of cotangents color (3,H,W), all_map (5,H,W), plane_depth (1,H,W).
    """
    W, H = cam["W"], cam["H"]
    gx, gy = tile_grid(W, H)
    if compute_locally is None:
        compute_locally = torch.ones(gy, gx, dtype=torch.bool)
    m2, dep, rad, cov3, co = preprocess_fwd(g["means3D"], g["scales"], g["rotations"], g["opacities"],
                                            cam["viewmatrix"], cam["projmatrix"], W, H, cam["tanfovx"], cam["tanfovy"])
    b = bin_and_sort(m2, dep, rad, compute_locally, W, H)
    f = render_fwd(m2, co, g["rgb"], g["all_map"], b["ranges"], b["point_list"], compute_locally, cam["bg"], W, H,
                   cam["tanfovx"], cam["tanfovy"], render_geo)
    out = dict(means2D=m2, depths=dep, radii=rad, cov3D=cov3, conic_opacity=co, **b, **f)
    if cot is not None:
        rb = render_bwd(m2, co, g["rgb"], g["all_map"], f["out_all_map"], f["final_T"], f["n_contrib_px"], b["ranges"],
                        b["point_list"], compute_locally, cam["bg"], W, H, cam["tanfovx"], cam["tanfovy"],
                        cot["color"], cot["all_map"], cot["plane_depth"], render_geo)
        pb = preprocess_bwd(g["means3D"], g["scales"], g["rotations"], rad, cov3, cam["viewmatrix"],
                            cam["projmatrix"], W, H, cam["tanfovx"], cam["tanfovy"], rb["dL_dmeans2D"],
                            rb["dL_dconic_opacity"])
        out.update(rb)
        out.update(pb)
    return out


def num_threads() -> int:
    return int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
