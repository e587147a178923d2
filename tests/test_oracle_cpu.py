"""CPU oracle: hand-checkable cases, internal consistency (finite differences), golden vectors."""
import math

import pytest
import torch

import util
from oracle import cpu_raster as O


def simple_camera(W=64, H=48):
    return util.S.look_at_camera(0, (0.0, 0.0, 10.0), (0.0, 0.0, 0.0), W, H, fov_x_deg=60.0, world_up=(0, 1, 0))


def test_higher_msb_and_key_layout():
    for n, want in [(1, 1), (144, 8), (7500, 13), (8160, 13), (32400, 15)]:
        assert O.higher_msb(n) == want
    cam = simple_camera()
    m2 = torch.tensor([[20.0, 20.0], [40.0, 30.0]])
    dep = torch.tensor([3.0, 1.5])
    rad = torch.tensor([3, 20], dtype=torch.int32)
    local = torch.ones(3, 4, dtype=torch.bool)
    b = O.bin_and_sort(m2, dep, rad, local, cam.W, cam.H)
    # gaussian 0: x in [17,23] -> tile 1, y in [17,23] -> tile 1: one tile (id 5); gaussian 1 covers tiles x 1..3, y 0..2
    assert b["tiles_touched"].tolist() == [1, 9]
    assert b["R"] == 10
    tiles = (b["keys"] >> 32).tolist()
    assert tiles == sorted(tiles)
    depth_bits = (b["keys"] & 0xFFFFFFFF).to(torch.int32).view(torch.float32)
    # tile 5 holds both; nearer (1.5) first
    sel = [i for i, t in enumerate(tiles) if t == 5]
    assert [b["point_list"][i].item() for i in sel] == [1, 0]
    assert depth_bits[sel[0]].item() == 1.5
    r = b["ranges"]
    assert r[5].tolist() == [sel[0], sel[-1] + 1]
    assert r[0].tolist() == [0, 0]          # tile 0 is empty -> (0,0)


def test_sort_is_stable_and_masks_high_bits():
    import ctypes as C
    n = 5000
    gen = torch.Generator().manual_seed(3)
    keys = torch.randint(0, 50, (n,), generator=gen, dtype=torch.int64) << 32
    keys |= torch.randint(0, 4, (n,), generator=gen, dtype=torch.int64)
    keys |= (torch.randint(0, 2, (n,), generator=gen, dtype=torch.int64) << 60)   # garbage above end_bit
    vals = torch.arange(n, dtype=torch.int32)
    ko, vo = torch.zeros_like(keys), torch.zeros_like(vals)
    O.lib().orc_sort_pairs(C.c_int64(n), 40, C.c_void_p(keys.data_ptr()), C.c_void_p(vals.data_ptr()),
                           C.c_void_p(ko.data_ptr()), C.c_void_p(vo.data_ptr()))
    masked = keys & ((1 << 40) - 1)
    order = torch.sort(masked, stable=True)[1]
    assert torch.equal(vo.long(), order)
    assert torch.equal(ko, keys[order])


def test_single_gaussian_closed_form():
    """One isotropic Gaussian in front of the camera: centre pixel alpha and colour follow from the formulas."""
    cam = simple_camera()
    s = 0.5
    g = dict(means3D=torch.tensor([[0.0, 0.0, 0.0]]), scales=torch.tensor([[s, s, s]]),
             rotations=torch.tensor([[1.0, 0.0, 0.0, 0.0]]), opacities=torch.tensor([[0.8]]),
             rgb=torch.tensor([[0.2, 0.5, 0.9]]), all_map=torch.tensor([[0.0, 0.0, 1.0, 1.0, 10.0]]))
    o = O.full_step(g, util.cam_dict(cam))
    f = cam.W / (2 * cam.tanfovx)
    var = (f * s / 10.0) ** 2 + 0.3
    assert o["radii"][0].item() == math.ceil(3 * math.sqrt(var))
    # projected centre: ((0+1)*W-1)/2
    cx, cy = (cam.W - 1) / 2, (cam.H - 1) / 2
    assert abs(o["means2D"][0, 0].item() - cx) < 1e-4 and abs(o["means2D"][0, 1].item() - cy) < 1e-4
    assert abs(o["depths"][0].item() - 10.0) < 1e-5
    px, py = 31, 23                      # nearest pixel to the centre: offset (0.5, 0.5)
    power = -0.5 * (0.25 + 0.25) / var
    alpha = 0.8 * math.exp(power)
    assert abs(o["color"][1, py, px].item() - 0.5 * alpha) < 1e-5
    assert abs(o["out_all_map"][3, py, px].item() - alpha) < 1e-5
    assert abs(o["final_T"].view(cam.H, cam.W)[py, px].item() - (1 - alpha)) < 1e-6
    # plane depth = distance / -(n.ray): normal (0,0,1) -> -(1) -> -10 * alpha / alpha-weighted... uses blended sums
    pd = o["out_plane_depth"][0, py, px].item()
    assert abs(pd - (10.0 * alpha) / -(alpha + 1e-8)) < 1e-4
    assert o["n_contrib_px"].view(cam.H, cam.W)[py, px].item() == 1


def test_culling_rules():
    cam = simple_camera()
    base = dict(scales=torch.full((3, 3), 0.1), rotations=torch.tensor([[1.0, 0, 0, 0]] * 3),
                opacities=torch.full((3, 1), 0.5))
    means = torch.tensor([[0.0, 0.0, 20.0],      # behind the camera (camera at z=10 looking down -z)
                          [0.0, 0.0, 10.0],      # exactly at the camera: z == 0 is culled (z <= 0)
                          [500.0, 0.0, 0.0]])    # far outside the image: no x/y frustum cull, but zero-area rect
    m2, dep, rad, cov3, co = O.preprocess_fwd(means, base["scales"], base["rotations"], base["opacities"],
                                              cam.viewmatrix, cam.projmatrix, cam.W, cam.H, cam.tanfovx, cam.tanfovy)
    assert rad.tolist() == [0, 0, 0]
    assert m2.abs().sum().item() == 0 and co.abs().sum().item() == 0
    assert cov3[0].abs().sum().item() == 0          # z-culled: covariance untouched
    assert cov3[2].abs().sum().item() > 0           # culled later: covariance already written


def _tiny_scene(n=40, res=(48, 32)):
    g, cam = util.make_case(cfg=1, n=n, res=res)
    g["means3D"] = g["means3D"] * 0.03
    g["scales"] = g["scales"] * 8
    g["all_map"] = util.S.build_all_map(g["means3D"], g["scales"], g["rotations"], cam)
    return g, cam


def test_backward_matches_finite_differences():
    """d(sum(out * cot))/d(param) from the oracle's backward vs central differences of its own forward.
    Restricted to opacities and colours, whose forward dependence is smooth (no radius / tile changes)."""
    g, cam = _tiny_scene()
    cot = util.cotangents(cam)
    cot["plane_depth"].zero_()          # 1/(n.ray) is too stiff for fp32 finite differences
    cd = util.cam_dict(cam)
    o = O.full_step(g, cd, cot=cot)

    def loss(gg):
        f = O.full_step(gg, cd)
        return float((f["color"].double() * cot["color"].double()).sum()
                     + (f["out_all_map"].double() * cot["all_map"].double()).sum())

    vis = torch.nonzero(o["out_observe"] > 0).flatten()[:6]
    assert len(vis) >= 3
    for i in vis.tolist():
        for name, gname, j in (("opacities", "dL_dopacity", 0), ("rgb", "dL_drgb", 1)):
            eps = 1e-2
            gp = {k: v.clone() for k, v in g.items()}
            gm = {k: v.clone() for k, v in g.items()}
            gp[name][i, j] += eps
            gm[name][i, j] -= eps
            fd = (loss(gp) - loss(gm)) / (2 * eps)
            an = o[gname][i, j].item()
            assert abs(fd - an) <= 2e-2 * max(1.0, abs(an)), (name, i, fd, an)


def test_preprocess_backward_matches_autograd_of_conic():
    """The fused preprocess backward against torch autograd (float64) of the same projection math."""
    g, cam = _tiny_scene(n=64)
    m2, dep, rad, cov3, co = O.preprocess_fwd(g["means3D"], g["scales"], g["rotations"], g["opacities"],
                                              cam.viewmatrix, cam.projmatrix, cam.W, cam.H, cam.tanfovx, cam.tanfovy)
    gen = torch.Generator().manual_seed(5)
    d_m2 = torch.randn(64, 2, generator=gen)
    d_co = torch.randn(64, 4, generator=gen)
    pb = O.preprocess_bwd(g["means3D"], g["scales"], g["rotations"], rad, cov3, cam.viewmatrix, cam.projmatrix,
                          cam.W, cam.H, cam.tanfovx, cam.tanfovy, d_m2, d_co)

    mean = g["means3D"].double().requires_grad_(True)
    sc = g["scales"].double().requires_grad_(True)
    q = g["rotations"].double().requires_grad_(True)
    V, Pm = cam.viewmatrix.double(), cam.projmatrix.double()
    r, x, y, z = q.unbind(-1)
    R = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - r * z), 2 * (x * z + r * y),
                     2 * (x * y + r * z), 1 - 2 * (x * x + z * z), 2 * (y * z - r * x),
                     2 * (x * z - r * y), 2 * (y * z + r * x), 1 - 2 * (x * x + y * y)], -1).view(-1, 3, 3)
    # the kernel lists these nine values column by column of a column-major matrix, i.e. it holds the transpose
    # of this (ordinary, row-listed) rotation matrix and forms (S R^T)^T (S R^T) = R S S R^T
    M = R @ torch.diag_embed(sc)
    Sigma = M @ M.transpose(1, 2)
    t = mean @ V[:3, :3] + V[3, :3]
    fx, fy = cam.W / (2 * cam.tanfovx), cam.H / (2 * cam.tanfovy)
    zero = torch.zeros_like(t[:, 0])
    J = torch.stack([fx / t[:, 2], zero, -fx * t[:, 0] / t[:, 2] ** 2,
                     zero, fy / t[:, 2], -fy * t[:, 1] / t[:, 2] ** 2], -1).view(-1, 2, 3)
    Wm = V[:3, :3].T
    T = J @ Wm
    cov = T @ Sigma @ T.transpose(1, 2)
    a, b, c = cov[:, 0, 0] + 0.3, cov[:, 0, 1], cov[:, 1, 1] + 0.3
    det = a * c - b * b
    conic = torch.stack([c / det, -b / det, a / det], -1)
    hom = torch.cat([mean, torch.ones_like(mean[:, :1])], 1) @ Pm
    ndc = hom[:, :2] / (hom[:, 3:4] + 1e-7)
    # pixel = ((ndc+1)*S-1)/2 -> d pixel = S/2 d ndc; the kernels fold S/2 into the render backward (ddelx_dx),
    # so the preprocess backward differentiates ndc, not pixels
    vis = rad > 0
    # convention of the rasterizer: the cotangent of the conic's off-diagonal term is the one of EACH of the two
    # symmetric matrix entries (the blending backward emits -0.5*dx*dy*dL_dG for it), hence the factor 2 here
    w = torch.tensor([1.0, 2.0, 1.0], dtype=torch.float64)
    lossv = (ndc[vis] * d_m2[vis].double()).sum() + (conic[vis] * w * d_co[vis, :3].double()).sum()
    lossv.backward()
    assert vis.sum() >= 20
    assert util.rel_l2(pb["dL_dmeans3D"][vis], mean.grad[vis].float()) < 1e-3
    assert util.rel_l2(pb["dL_dscales"][vis], sc.grad[vis].float()) < 1e-3
    assert util.rel_l2(pb["dL_drotations"][vis], q.grad[vis].float()) < 1e-3
    assert torch.equal(pb["dL_dopacity"][:, 0], d_co[:, 3])
    assert pb["dL_dmeans3D"][~vis].abs().sum().item() == 0


def test_local2j_mask_semantics():
    cam = simple_camera(W=64, H=64)          # 4x4 tiles
    m2 = torch.tensor([[8.0, 8.0], [8.0, 31.0], [40.0, 40.0], [0.0, 0.0]])
    rad = torch.tensor([2, 3, 30, 0], dtype=torch.int32)
    bounds = torch.tensor([0, 2, 4], dtype=torch.int32) * 4       # two ranks, two tile rows each
    mask = O.local2j_mask(m2, rad, bounds, 64, 64)
    assert mask.tolist() == [[True, False],        # inside row 0
                             [True, True],         # y span 28..34 straddles the cut at y=32
                             [True, True],         # huge splat
                             [False, False]]       # culled row (means2D = 0, radius 0): empty span


GOLDEN_FILES = sorted(util.GOLDEN.glob("cfg*.npz"))     # rasterizer cases (the loss cases are loss_*.npz)


@pytest.mark.parametrize("path", GOLDEN_FILES, ids=lambda p: p.stem)
def test_oracle_against_reference_golden(path):
    """Outputs of the reference's own CUDA extension (captured on a B200 by tests/golden/make_golden.py)."""
    import numpy as np

    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files}
    case = {k: (int(v) if v.numel() == 1 else tuple(int(x) for x in v)) for k, v in t.items() if k.startswith("case_")}
    g, cam = util.make_case(cfg=case["case_cfg"], n=case["case_n"], res=case["case_res"],
                            big_scales=bool(case.get("case_big", 0)))
    cot = util.cotangents(cam)
    cd = util.cam_dict(cam)
    m2, dep, rad, cov3, co, fragile = O.preprocess_fwd(g["means3D"], g["scales"], g["rotations"], g["opacities"],
                                                       cam.viewmatrix, cam.projmatrix, cam.W, cam.H, cam.tanfovx,
                                                       cam.tanfovy, want_fragile=True)
    ok = ~fragile
    assert torch.equal(rad[ok], t["radii"][ok])
    assert (rad != t["radii"]).float().mean().item() < 1e-4
    vis = ok & (rad > 0)
    assert (m2[vis] - t["means2D"][vis]).abs().max().item() < 2e-3
    # binning / blending / backward are pinned stage by stage on the reference's own inputs to each stage
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    local = torch.ones(TY, TX, dtype=torch.bool)
    b = O.bin_and_sort(t["means2D"], t["depths"], t["radii"], local, cam.W, cam.H)
    assert b["R"] == int(t["R"])
    assert torch.equal(b["keys"], t["keys"]) and torch.equal(b["point_list"], t["point_list"])
    assert torch.equal(b["ranges"], t["ranges"])
    f = O.render_fwd(t["means2D"], t["conic_opacity"], g["rgb"], g["all_map"], t["ranges"], t["point_list"], local,
                     cd["bg"], cam.W, cam.H, cam.tanfovx, cam.tanfovy)
    for k in ("color", "out_all_map"):
        assert ((f[k] - t[k]).abs() > 2e-5).float().mean().item() < 1e-4, k
    assert (f["n_contrib_px"] != t["n_contrib_px"]).float().mean().item() < 1e-4
    rb = O.render_bwd(t["means2D"], t["conic_opacity"], g["rgb"], g["all_map"], t["out_all_map"], t["final_T"],
                      t["n_contrib_px"], t["ranges"], t["point_list"], local, cd["bg"], cam.W, cam.H, cam.tanfovx,
                      cam.tanfovy, cot["color"], cot["all_map"], cot["plane_depth"])
    for k in ("dL_dmeans2D", "dL_drgb", "dL_dall_map"):
        assert util.rel_l2(rb[k], t[k]) < 2e-3, (k, util.rel_l2(rb[k], t[k]))
    pb = O.preprocess_bwd(g["means3D"], g["scales"], g["rotations"], t["radii"], t["cov3D"], cam.viewmatrix,
                          cam.projmatrix, cam.W, cam.H, cam.tanfovx, cam.tanfovy, t["dL_dmeans2D"],
                          rb["dL_dconic_opacity"])
    for k in ("dL_dmeans3D", "dL_dscales", "dL_drotations"):
        assert util.rel_l2(pb[k], t[k]) < 3e-3, (k, util.rel_l2(pb[k], t[k]))
