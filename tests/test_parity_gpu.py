"""GPU parity: the CUDA path (through the C ABI / drop-in package) against

  (1) the reference's own CUDA extension on identical inputs, when it is available (built by
      oracle/build_ref.py): radii, sorted keys, point list, tile ranges, n_contrib bit-exact; forward images
      within 1e-5 max-abs; gradients within 1e-3 relative L2;
  (2) the CPU oracle: integer stages exactly (each stage fed with the GPU's own inputs to it), float stages
      within tolerance.
"""
import pytest
import torch

import util
from util import cam_dict, cotangents, cuda_args, decode_binning, decode_image, make_case, rel_l2, settings_for

pytestmark = pytest.mark.gpu

FWD_TOL = 1e-5      # max-abs on forward images (north-star tolerance)
GRAD_TOL = 1e-3     # relative L2 on every gradient tensor, CUDA path vs the reference's CUDA rasterizer
# Against the CPU oracle the bar is looser: it accumulates in double and uses libm's expf, the device sums fp32
# atomics in arbitrary order and uses its own expf, and the plane-depth cotangent (1/(n.ray)^2) amplifies both.
ORACLE_GRAD_TOL = 5e-3

CASES = [
    dict(cfg=1, n=20000, res=(320, 180)),
    dict(cfg=1, n=200000, res=(640, 360)),
    dict(cfg=0, n=50000, res=(256, 144)),
    dict(cfg=1, n=30000, res=(333, 211), big_scales=True),     # not multiples of 16, many tiles per splat
    dict(cfg=2, n=300000, res=(800, 600)),
    # the named configurations at their own resolution: 1M Gaussians at 1920x1080 (8160 tiles, 45 key bits), and
    # the clustered city on a 3840x2160 grid (32400 tiles -> 15 tile bits, 47 key bits) with a reduced Gaussian count
    dict(cfg=1, n=1_000_000, res=(1920, 1080)),
    dict(cfg=3, n=2_000_000, res=(3840, 2160), cam_idx=5),
]


def to_dev(g, dev):
    return {k: v.to(dev) for k, v in g.items()}


def run_ours(g, cam, dev, local=None, cot=None, render_geo=True, bg=None, debug=True):
    """Full path through the drop-in package. Returns dict of CPU tensors."""
    from diff_gaussian_rasterization import GaussianRasterizer, _C

    rs = settings_for(cam, dev, bg=bg, render_geo=render_geo, debug=debug)
    rast = GaussianRasterizer(rs)
    gd = to_dev(g, dev)
    leaves = {}
    for k in ("means3D", "scales", "rotations", "opacities", "rgb", "all_map"):
        leaves[k] = gd[k].clone().requires_grad_(cot is not None)
    args = cuda_args()
    means2D, rgb0, conic_opacity, radii, depths = rast.preprocess_gaussians(
        leaves["means3D"], leaves["scales"], leaves["rotations"], gd["sh"], leaves["opacities"], args)
    if cot is not None:
        means2D.retain_grad()
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    if local is None:
        local = torch.ones(TY, TX, dtype=torch.bool)
    local_d = local.to(dev)
    means2D_abs = torch.zeros(means2D.shape[0], 3, device=dev, requires_grad=cot is not None)
    # raw call as well, to look at the scratch buffers
    raw = _C.render_gaussians(rs.bg, cam.H, cam.W, means2D.detach(), depths, radii, conic_opacity.detach(),
                              leaves["rgb"].detach(), local_d, rs.viewmatrix, rs.campos, cam.tanfovx, cam.tanfovy,
                              leaves["all_map"].detach(), render_geo, True, args)
    R = raw[0]
    bn = decode_binning(raw[9], R) if R else None
    im = decode_image(raw[10], cam.W * cam.H, TX * TY) if means2D.shape[0] else None
    color, n_render, n_consider, n_contrib, observe, out_all_map, plane_depth = rast.render_gaussians(
        means2D, means2D_abs, conic_opacity, leaves["rgb"], leaves["all_map"], depths, radii, local_d, None, args)
    out = dict(means2D=means2D, depths=depths, radii=radii, conic_opacity=conic_opacity, R=R, color=color,
               n_render=n_render, n_consider=n_consider, n_contrib=n_contrib, out_observe=observe,
               out_all_map=out_all_map, out_plane_depth=plane_depth)
    if bn is not None:
        out.update(keys=bn["point_list_keys"], point_list=bn["point_list"], keys_unsorted=None)
    if im is not None:
        out.update(ranges=im["ranges"].view(-1, 2), final_T=im["accum_alpha"], n_contrib_px=im["n_contrib"],
                   n_contrib2loss_px=im["n_contrib2loss"])
    if cot is not None:
        loss = ((color * cot["color"].to(dev)).sum() + (out_all_map * cot["all_map"].to(dev)).sum()
                + (plane_depth * cot["plane_depth"].to(dev)).sum())
        loss.backward()
        out.update(dL_dmeans3D=leaves["means3D"].grad, dL_dscales=leaves["scales"].grad,
                   dL_drotations=leaves["rotations"].grad, dL_dopacity=leaves["opacities"].grad,
                   dL_drgb=leaves["rgb"].grad, dL_dall_map=leaves["all_map"].grad, dL_dmeans2D=means2D.grad,
                   dL_dmeans2D_abs=means2D_abs.grad)
    torch.cuda.synchronize()
    return {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in out.items()}


def run_reference(ref, g, cam, dev, local=None, cot=None, render_geo=True, bg=None):
    """Same path through the reference extension's raw entry points."""
    gd = to_dev(g, dev)
    V, Pm, campos = cam.viewmatrix.to(dev), cam.projmatrix.to(dev), cam.campos.to(dev)
    bgd = (torch.zeros(3) if bg is None else bg).to(dev)
    args = cuda_args()
    _, means2D, depths, radii, cov3D, conic_opacity, rgb0, clamped = ref.preprocess_gaussians(
        gd["means3D"], gd["scales"], gd["rotations"], gd["sh"], gd["opacities"], 1.0, V, Pm, cam.tanfovx, cam.tanfovy,
        cam.H, cam.W, 3, campos, False, False, args)
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    if local is None:
        local = torch.ones(TY, TX, dtype=torch.bool)
    local_d = local.to(dev)
    (R, color, n_render, n_consider, n_contrib, observe, out_all_map, plane_depth, geomB, binB, imgB) = \
        ref.render_gaussians(bgd, cam.H, cam.W, means2D, depths, radii, conic_opacity, gd["rgb"], local_d, V, campos,
                             cam.tanfovx, cam.tanfovy, gd["all_map"], render_geo, False, args)
    out = dict(means2D=means2D, depths=depths, radii=radii, conic_opacity=conic_opacity, cov3D=cov3D, R=R,
               color=color, n_render=n_render, n_consider=n_consider, n_contrib=n_contrib, out_observe=observe,
               out_all_map=out_all_map, out_plane_depth=plane_depth)
    if R:
        bn = decode_binning(binB, R)
        out.update(keys=bn["point_list_keys"], point_list=bn["point_list"])
    im = decode_image(imgB, cam.W * cam.H, cam.W * cam.H)
    out.update(ranges=im["ranges"].view(-1, 2)[: TX * TY], final_T=im["accum_alpha"], n_contrib_px=im["n_contrib"],
               n_contrib2loss_px=im["n_contrib2loss"])
    if cot is not None:
        d_m2, d_abs, d_co, d_rgb, d_map = ref.render_gaussians_backward(
            bgd, cam.tanfovx, cam.tanfovy, out_all_map, gd["all_map"], R, geomB, binB, imgB, local_d,
            cot["color"].to(dev), cot["all_map"].to(dev), cot["plane_depth"].to(dev), means2D, conic_opacity,
            gd["rgb"], render_geo, False, args)
        d_means, d_scales, d_rot, d_sh, d_op = ref.preprocess_gaussians_backward(
            radii, cov3D, clamped, gd["means3D"], gd["scales"], gd["rotations"], gd["sh"], 1.0, V, Pm, cam.tanfovx,
            cam.tanfovy, cam.H, cam.W, 3, campos, d_m2.contiguous(), d_co, torch.zeros_like(gd["rgb"]), R, False, args)
        out.update(dL_dmeans3D=d_means, dL_dscales=d_scales, dL_drotations=d_rot, dL_dopacity=d_op, dL_drgb=d_rgb,
                   dL_dall_map=d_map, dL_dmeans2D=d_m2[:, :2], dL_dmeans2D_abs=d_abs)
    torch.cuda.synchronize()
    return {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in out.items()}


GRADS = ["dL_dmeans3D", "dL_dscales", "dL_drotations", "dL_dopacity", "dL_drgb", "dL_dall_map", "dL_dmeans2D",
         "dL_dmeans2D_abs"]


def masked_local(x, cam, local):
    """Zero pixels of tiles that are not computed locally (the reference leaves no defined value contractually,
    but both sides zero them; compare only local pixels to be safe)."""
    if local is None:
        return x
    m = local.repeat_interleave(16, 0).repeat_interleave(16, 1)[: cam.H, : cam.W]
    return x * m


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"cfg{c['cfg']}-{c['n']}-{c['res'][0]}x{c['res'][1]}")
def test_against_reference_extension(case, cuda_device, reference_C):
    assert reference_C is not None, "oracle/_ref/cityx_ref_C.so is missing: build it with oracle/build_ref.py"
    g, cam = make_case(**case)
    cot = cotangents(cam)
    ours = run_ours(g, cam, cuda_device, cot=cot)
    ref = run_reference(reference_C, g, cam, cuda_device, cot=cot)
    # --- bit-exact integers and the floats they derive from
    assert torch.equal(ours["radii"], ref["radii"])
    assert torch.equal(ours["means2D"], ref["means2D"])
    assert torch.equal(ours["depths"], ref["depths"])
    assert torch.equal(ours["conic_opacity"], ref["conic_opacity"])
    assert ours["R"] == ref["R"] and ours["R"] > 0
    assert torch.equal(ours["keys"], ref["keys"])
    assert torch.equal(ours["point_list"], ref["point_list"])
    assert torch.equal(ours["ranges"], ref["ranges"])
    assert torch.equal(ours["n_contrib_px"], ref["n_contrib_px"])
    assert torch.equal(ours["n_contrib2loss_px"], ref["n_contrib2loss_px"])
    for k in ("n_render", "n_consider", "n_contrib", "out_observe"):
        assert torch.equal(ours[k], ref[k]), k
    # --- forward images
    for k in ("color", "out_all_map", "final_T"):
        assert (ours[k] - ref[k]).abs().max().item() <= FWD_TOL, k
    pd_o, pd_r = ours["out_plane_depth"], ref["out_plane_depth"]
    big = pd_r.abs() > 1e3          # 1/(n.ray) is unbounded at grazing normals: relative there
    assert ((pd_o - pd_r).abs()[~big]).max().item() <= FWD_TOL * 10
    if big.any():
        assert (((pd_o - pd_r).abs() / pd_r.abs())[big]).max().item() <= 1e-5
    # --- gradients
    for k in GRADS:
        assert rel_l2(ours[k], ref[k]) <= GRAD_TOL, (k, rel_l2(ours[k], ref[k]))


@pytest.mark.parametrize("case", CASES[:4], ids=lambda c: f"cfg{c['cfg']}-{c['n']}-{c['res'][0]}x{c['res'][1]}")
def test_against_cpu_oracle(case, cuda_device):
    from oracle import cpu_raster as O

    g, cam = make_case(**case)
    cot = cotangents(cam)
    ours = run_ours(g, cam, cuda_device, cot=cot)
    cd = cam_dict(cam)
    # stage 1: preprocess. The CPU does not contract multiply-adds, so integers are compared where the
    # oracle says the input is not within rounding distance of a boundary.
    m2, dep, rad, cov3, co, fragile = O.preprocess_fwd(g["means3D"], g["scales"], g["rotations"], g["opacities"],
                                                       cam.viewmatrix, cam.projmatrix, cam.W, cam.H, cam.tanfovx,
                                                       cam.tanfovy, want_fragile=True)
    ok = ~fragile
    assert fragile.float().mean().item() < 0.02
    assert torch.equal(ours["radii"][ok], rad[ok])
    vis = ok & (rad > 0)
    assert (ours["means2D"][vis] - m2[vis]).abs().max().item() < 2e-3
    assert rel_l2(ours["conic_opacity"][vis], co[vis]) < 1e-4
    assert rel_l2(ours["depths"][vis], dep[vis]) < 1e-6
    # stage 2: binning on the GPU's own preprocess outputs -> exact
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    local = torch.ones(TY, TX, dtype=torch.bool)
    b = O.bin_and_sort(ours["means2D"], ours["depths"], ours["radii"], local, cam.W, cam.H)
    assert b["R"] == ours["R"]
    assert torch.equal(b["keys"], ours["keys"])
    assert torch.equal(b["point_list"], ours["point_list"])
    assert torch.equal(b["ranges"], ours["ranges"])
    # stage 3: blending on the GPU's own lists
    f = O.render_fwd(ours["means2D"], ours["conic_opacity"], g["rgb"], g["all_map"], ours["ranges"],
                     ours["point_list"], local, cd["bg"], cam.W, cam.H, cam.tanfovx, cam.tanfovy)
    # libm expf and the device expf differ in the last bits: a pixel whose alpha sits on the 1/255 threshold can
    # flip, so allow a tiny fraction of outlier pixels
    for k in ("color", "out_all_map"):
        bad = ((ours[k] - f[k]).abs() > 2e-5).float().mean().item()
        assert bad < 1e-4, (k, bad)
    mism = (ours["n_contrib_px"] != f["n_contrib_px"]).float().mean().item()
    assert mism < 1e-4
    # stage 4: backward on the GPU's own forward state
    rb = O.render_bwd(ours["means2D"], ours["conic_opacity"], g["rgb"], g["all_map"], ours["out_all_map"],
                      ours["final_T"], ours["n_contrib_px"], ours["ranges"], ours["point_list"], local, cd["bg"],
                      cam.W, cam.H, cam.tanfovx, cam.tanfovy, cot["color"], cot["all_map"], cot["plane_depth"])
    for k in ("dL_dmeans2D", "dL_dmeans2D_abs", "dL_drgb", "dL_dall_map"):
        assert rel_l2(ours[k], rb[k]) <= ORACLE_GRAD_TOL, (k, rel_l2(ours[k], rb[k]))
    pb = O.preprocess_bwd(g["means3D"], g["scales"], g["rotations"], ours["radii"], cov3, cam.viewmatrix,
                          cam.projmatrix, cam.W, cam.H, cam.tanfovx, cam.tanfovy, ours["dL_dmeans2D"],
                          rb["dL_dconic_opacity"])
    for k in ("dL_dmeans3D", "dL_dscales", "dL_drotations", "dL_dopacity"):
        assert rel_l2(ours[k], pb[k]) <= ORACLE_GRAD_TOL, (k, rel_l2(ours[k], pb[k]))


def test_reference_extension_is_present(reference_C):
    """The parity tests above are only as good as their checker: a box without the reference's compiled extension
    must fail, not skip."""
    assert reference_C is not None, "oracle/_ref/cityx_ref_C.so is missing: build it with oracle/build_ref.py"
    assert reference_C.get_block_XY() == (16, 16, 256)


def test_stats_collector_gets_render_times(cuda_device):
    """The op fills args["stats_collector"] with the forward and backward blending times in milliseconds
    (cuda_rasterizer/rasterizer_impl.cu:754-755, 924-926); the balancer divides work by them."""
    from diff_gaussian_rasterization import GaussianRasterizer

    g, cam = make_case(cfg=2, n=100_000, res=(640, 480))
    dev = cuda_device
    rast = GaussianRasterizer(settings_for(cam, dev))
    gd = to_dev(g, dev)
    stats = {}
    args = cuda_args(stats)
    m2, _, co, radii, depths = rast.preprocess_gaussians(gd["means3D"].requires_grad_(True), gd["scales"],
                                                         gd["rotations"], gd["sh"], gd["opacities"], args)
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    local = torch.ones(TY, TX, dtype=torch.bool, device=dev)
    m2abs = torch.zeros(m2.shape[0], 3, device=dev, requires_grad=True)
    color, *_ = rast.render_gaussians(m2, m2abs, co, gd["rgb"], gd["all_map"], depths, radii, local, None, args)
    assert "forward_render_time" in stats and "backward_render_time" not in stats
    color.sum().backward()
    fwd, bwd = float(stats["forward_render_time"]), float(stats["backward_render_time"])
    assert 0.0 < fwd < 1000.0 and 0.0 < bwd < 1000.0
    assert stats["forward_render_time"] + stats["backward_render_time"] == pytest.approx(fwd + bwd)


def test_cull_variant_is_identical(cuda_device):
    """Per-warp culling and the two-phase walk must not change a single bit of the forward outputs, and the
    gradients only by the order of their sums."""
    from diff_gaussian_rasterization import _lib

    g, cam = make_case(cfg=1, n=100000, res=(640, 360), big_scales=True)
    l = _lib.lib()
    try:
        l.cgx_set_render_variant(1)      # default: culling, walk chosen from the measured density
        a = run_ours(g, cam, cuda_device, cot=cotangents(cam))
        l.cgx_set_render_variant(0)      # no culling, every lane looks at every Gaussian
        b = run_ours(g, cam, cuda_device, cot=cotangents(cam))
        l.cgx_set_render_variant(3)      # culling, every lane looks at every surviving Gaussian
        c = run_ours(g, cam, cuda_device, cot=cotangents(cam))
        l.cgx_set_render_variant(5)      # culling, two-phase walk whatever the density
        e = run_ours(g, cam, cuda_device, cot=cotangents(cam))
    finally:
        l.cgx_set_render_variant(1)
    for k in ("color", "out_all_map", "out_plane_depth", "final_T", "n_contrib_px", "n_contrib2loss_px",
              "out_observe", "n_consider", "n_contrib"):
        assert torch.equal(a[k], b[k]), k
        assert torch.equal(a[k], c[k]), k
        assert torch.equal(a[k], e[k]), k
    for k in GRADS:
        assert rel_l2(a[k], b[k]) <= 1e-5, k
        assert rel_l2(a[k], c[k]) <= 1e-5, k
        assert rel_l2(a[k], e[k]) <= 1e-5, k


@pytest.mark.parametrize("shape", ["band", "scattered", "none"])
def test_partial_compute_locally(shape, cuda_device, reference_C):
    """Only some tiles are local: keys only for local tiles, other pixels zero.  A band of whole tile rows (what the
    workload division produces) takes the library's row-band shortcut, scattered tiles the per-tile lookups."""
    from oracle import cpu_raster as O

    g, cam = make_case(cfg=1, n=50000, res=(640, 360))
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    local = torch.zeros(TY, TX, dtype=torch.bool)
    if shape == "band":
        local[5:13] = True
    elif shape == "scattered":
        local[:] = torch.rand(TY, TX, generator=torch.Generator().manual_seed(5)) > 0.5
        local[7] = True          # a full row among partial ones
    cot = cotangents(cam)
    ours = run_ours(g, cam, cuda_device, local=local, cot=cot)
    if shape == "none":
        assert ours["R"] == 0 and ours["color"].abs().max().item() == 0.0
        return
    b = O.bin_and_sort(ours["means2D"], ours["depths"], ours["radii"], local, cam.W, cam.H)
    assert b["R"] == ours["R"]
    assert torch.equal(b["keys"], ours["keys"]) and torch.equal(b["point_list"], ours["point_list"])
    assert torch.equal(b["ranges"], ours["ranges"])
    m = local.repeat_interleave(16, 0).repeat_interleave(16, 1)[: cam.H, : cam.W]
    assert ours["color"][:, ~m].abs().max().item() == 0.0
    assert ours["out_all_map"][:, ~m].abs().max().item() == 0.0
    if reference_C is not None:
        ref = run_reference(reference_C, g, cam, cuda_device, local=local, cot=cot)
        assert torch.equal(ours["keys"], ref["keys"]) and torch.equal(ours["ranges"], ref["ranges"])
        assert (ours["color"] - ref["color"]).abs().max().item() <= FWD_TOL
        for k in GRADS:
            assert rel_l2(ours[k], ref[k]) <= GRAD_TOL, k


@pytest.mark.parametrize("P", [0, 1, 31, 32, 33, 255, 257])
def test_small_counts(P, cuda_device):
    from oracle import cpu_raster as O

    g, cam = make_case(cfg=1, n=max(P, 1), res=(64, 48))
    g = {k: v[:P].contiguous() for k, v in g.items()}
    # pull everything in front of the camera so tiny P still renders something
    g["means3D"] = g["means3D"] * 0.05
    g["scales"] = g["scales"] * 5
    g["all_map"] = util.S.build_all_map(g["means3D"], g["scales"], g["rotations"], cam)
    cot = cotangents(cam)
    ours = run_ours(g, cam, cuda_device, cot=cot if P else None)
    assert ours["color"].shape == (3, cam.H, cam.W)
    assert ours["radii"].shape == (P,)
    if P == 0:
        assert ours["color"].abs().max().item() == 0
        return
    cd = cam_dict(cam)
    o = O.full_step(dict(g), cd, cot=cot)
    assert torch.equal(ours["radii"], o["radii"])
    assert (ours["color"] - o["color"]).abs().max().item() < 1e-4
    for k in GRADS:
        if k in o:
            assert rel_l2(ours[k], o[k]) <= 5e-3, (k, rel_l2(ours[k], o[k]))


def test_all_culled_and_background(cuda_device):
    g, cam = make_case(cfg=1, n=1000, res=(96, 64))
    g["means3D"][:, :] = torch.tensor([0.0, -200.0, 200.0])     # behind the camera
    bg = torch.tensor([0.25, 0.5, 0.75])
    ours = run_ours(g, cam, cuda_device, bg=bg)
    assert (ours["radii"] == 0).all() and ours["R"] == 0
    assert torch.allclose(ours["color"], bg[:, None, None].expand(3, cam.H, cam.W))
    assert (ours["final_T"] == 1).all()


def test_filter_and_mark_visible(cuda_device, reference_C):
    from diff_gaussian_rasterization import GaussianRasterizer
    from oracle import cpu_raster as O

    g, cam = make_case(cfg=1, n=100000, res=(640, 360))
    rast = GaussianRasterizer(settings_for(cam, cuda_device))
    gd = to_dev(g, cuda_device)
    radii_f = rast.visible_filter(gd["means3D"], gd["scales"], gd["rotations"]).cpu()
    vis = rast.markVisible(gd["means3D"]).cpu()
    m2, dep, rad, cov3, co, fragile = O.preprocess_fwd(g["means3D"], g["scales"], g["rotations"], g["opacities"],
                                                       cam.viewmatrix, cam.projmatrix, cam.W, cam.H, cam.tanfovx,
                                                       cam.tanfovy, want_fragile=True)
    assert torch.equal(radii_f[~fragile], rad[~fragile])
    assert (vis != O.mark_visible(g["means3D"], cam.viewmatrix)).float().mean().item() < 1e-4
    ours = run_ours(g, cam, cuda_device)
    assert torch.equal(radii_f, ours["radii"])        # same geometry as the full preprocess, bit for bit
    if reference_C is not None:
        V, Pm = cam.viewmatrix.to(cuda_device), cam.projmatrix.to(cuda_device)
        r_ref = reference_C.rasterize_aussians_filter(gd["means3D"], gd["scales"], gd["rotations"], 1.0,
                                                      torch.empty(0, device=cuda_device), V, Pm, cam.tanfovx,
                                                      cam.tanfovy, cam.H, cam.W, False, False).cpu()
        assert torch.equal(radii_f, r_ref)
        assert torch.equal(vis, reference_C.mark_visible(gd["means3D"], V, Pm).cpu())
    # precomputed 3-D covariances instead of scales and rotations (forward.cu:585-595): same radii
    from diff_gaussian_rasterization import _C
    rs = rast.raster_settings
    cov3D = _C.preprocess_gaussians(gd["means3D"], gd["scales"], gd["rotations"], gd["sh"], gd["opacities"], 1.0,
                                    rs.viewmatrix, rs.projmatrix, cam.tanfovx, cam.tanfovy, cam.H, cam.W, 3, rs.campos,
                                    False, False, cuda_args())[4]
    radii_c = rast.visible_filter(gd["means3D"], cov3D_precomp=cov3D).cpu()
    assert torch.equal(radii_c, radii_f)
    if reference_C is not None:
        e = torch.empty(0, device=cuda_device)
        r_ref_c = reference_C.rasterize_aussians_filter(gd["means3D"], e, e, 1.0, cov3D, V, Pm, cam.tanfovx, cam.tanfovy,
                                                        cam.H, cam.W, False, False).cpu()
        assert torch.equal(radii_c, r_ref_c)


def test_sh_stage(cuda_device):
    import ctypes as C

    from diff_gaussian_rasterization import _lib
    from oracle import cpu_raster as O

    g, cam = make_case(cfg=1, n=5000, res=(64, 48))
    dev = cuda_device
    P = g["means3D"].shape[0]
    rgb = torch.empty(P, 3, device=dev)
    clamped = torch.empty(P, 3, dtype=torch.bool, device=dev)
    m, sh, cp = g["means3D"].to(dev), g["sh"].to(dev), cam.campos.to(dev)
    for deg in range(4):
        st = _lib.lib().cgx_sh_to_rgb(P, deg, 16, m.data_ptr(), cp.data_ptr(), sh.data_ptr(), rgb.data_ptr(),
                                      clamped.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0
        ref_rgb, ref_cl = O.sh_to_rgb(g["means3D"], cam.campos, g["sh"], deg)
        assert (rgb.cpu() - ref_rgb).abs().max().item() < 1e-5
        assert (clamped.cpu() != ref_cl).float().mean().item() < 1e-3


def test_error_codes(cuda_device):
    from diff_gaussian_rasterization import GaussianRasterizer, _lib

    g, cam = make_case(cfg=1, n=100, res=(64, 48))
    rast = GaussianRasterizer(settings_for(cam, cuda_device))
    gd = to_dev(g, cuda_device)
    with pytest.raises(RuntimeError):
        rast.preprocess_gaussians(gd["means3D"][:, :2], gd["scales"], gd["rotations"], gd["sh"], gd["opacities"],
                                  cuda_args())
    with pytest.raises(RuntimeError):      # CPU tensors are refused, never silently computed on the host
        rast.preprocess_gaussians(g["means3D"], g["scales"], g["rotations"], g["sh"], g["opacities"], cuda_args())
    l = _lib.lib()
    assert l.cgx_preprocess_fwd(-1, *([None] * 2), 1.0, *([None] * 4), 64, 48, 0.5, 0.5, *([None] * 6)) == _lib.CGX_EINVAL
    assert l.cgx_sort_pairs(10, 40, None, None, None, None, None, 0, None) == _lib.CGX_EINVAL
    from diff_gaussian_rasterization import _C
    with pytest.raises(RuntimeError, match="deprecated"):
        _C.get_distribution_strategy(48, 64, None, None, False, {})


def test_batched_preprocess_equals_per_camera(cuda_device):
    """The camera-batched operator: per-camera outputs bit-identical, summed gradients within tolerance."""
    from cgx.batched import preprocess_gaussians_batched
    from diff_gaussian_rasterization import GaussianRasterizer

    g, cams = util.S.config(2, n_gaussians=60000, n_cameras=5, res=(320, 240))
    dev = cuda_device
    settings = [settings_for(c, dev) for c in cams]
    gen = torch.Generator().manual_seed(3)
    cot = [(torch.randn(60000, 2, generator=gen).to(dev), torch.randn(60000, 4, generator=gen).to(dev)) for _ in cams]

    def leaves():
        return [g[k].to(dev).clone().requires_grad_(True) for k in ("means3D", "scales", "rotations", "opacities")]

    a = leaves()
    outs_a = [GaussianRasterizer(s).preprocess_gaussians(a[0], a[1], a[2], torch.empty(0, device=dev), a[3], cuda_args())
              for s in settings]
    b = leaves()
    outs_b = preprocess_gaussians_batched(b[0], b[1], b[2], torch.empty(0, device=dev), b[3], settings, cuda_args())
    for (m2a, _, coa, ra, da), (m2b, _, cob, rb, db) in zip(outs_a, outs_b):
        assert torch.equal(m2a, m2b) and torch.equal(coa, cob) and torch.equal(ra, rb) and torch.equal(da, db)
    # camera 3 gets no cotangent at all: it must simply not contribute
    heads_a, heads_b, gr = [], [], []
    for k in range(len(cams)):
        if k == 3:
            continue
        heads_a += [outs_a[k][0], outs_a[k][2]]
        heads_b += [outs_b[k][0], outs_b[k][2]]
        gr += list(cot[k])
    torch.autograd.backward(heads_a, gr)
    torch.autograd.backward(heads_b, gr)
    for x, y in zip(a, b):
        assert rel_l2(y.grad.cpu(), x.grad.cpu()) <= 1e-5


@pytest.mark.parametrize("n,end_bit", [(1, 45), (255, 45), (4096, 45), (4097, 45), (1_000_003, 45), (300_007, 47),
                                       (70_001, 40), (5000, 33), (2_500_000, 47)])
def test_sort_pairs_variants(n, end_bit, cuda_device):
    """Both three-kernel scatter strategies and the one-sweep passes: identical output, equal to a stable sort on
    the masked key; through the copy-free ping-pong entry point and through the in -> out one."""
    import ctypes as C

    from diff_gaussian_rasterization import _lib

    l = _lib.lib()
    dev = cuda_device
    gen = torch.Generator().manual_seed(n)
    tiles = 32400 if end_bit == 47 else 8160
    keys = (torch.randint(0, tiles, (n,), generator=gen, dtype=torch.int64) << 32) | \
        torch.randint(0, 1 << 32, (n,), generator=gen, dtype=torch.int64)
    # few distinct depths in a part of the array: long runs of equal keys test stability
    keys[: n // 3] &= ~torch.tensor(0xFFFFF, dtype=torch.int64)
    keys |= torch.randint(0, 2, (n,), generator=gen, dtype=torch.int64) << 50       # above end_bit: must be ignored
    vals = torch.arange(n, dtype=torch.int32)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    order = torch.sort(keys & ((1 << end_bit) - 1), stable=True)[1]
    passes = l.cgx_sort_passes(end_bit)
    assert passes == (end_bit + 7) // 8
    try:
        for variant in (-1, 0, 1, 2):
            l.cgx_set_sort_variant(variant)
            ws = torch.empty(l.cgx_sort_workspace_bytes(n), dtype=torch.uint8, device=dev)
            kin, vin = keys.to(dev), vals.to(dev)
            kout, vout = torch.empty_like(kin), torch.empty_like(vin)
            assert l.cgx_sort_pairs(n, end_bit, kin.data_ptr(), vin.data_ptr(), kout.data_ptr(), vout.data_ptr(),
                                    ws.data_ptr(), ws.numel(), st) == 0
            torch.cuda.synchronize()
            assert torch.equal(vout.cpu().long(), order) and torch.equal(kout.cpu(), keys[order]), variant
            ka, va = keys.to(dev), vals.to(dev)
            kb, vb = torch.zeros_like(ka), torch.zeros_like(va)
            assert l.cgx_sort_pairs_pingpong(n, end_bit, 32, ka.data_ptr(), va.data_ptr(), kb.data_ptr(),
                                             vb.data_ptr(), ws.data_ptr(), ws.numel(), 0, st) == 0
            torch.cuda.synchronize()
            k, v = (ka, va) if passes % 2 == 0 else (kb, vb)
            assert torch.equal(v.cpu().long(), order) and torch.equal(k.cpu(), keys[order]), variant
            if end_bit > 32:
                # keys whose depth words share their 7 leading bits (as the depths of one view do): the sort is told
                # so and runs over 25 + tile bits, the keys travel unchanged and the order is that of the full sort
                low = 25
                shared = (keys & ~torch.tensor(0xFE000000, dtype=torch.int64)) | 0x42000000
                want = torch.sort(shared & ((1 << end_bit) - 1), stable=True)[1]
                ka, va = shared.to(dev), vals.to(dev)
                kb, vb = torch.zeros_like(ka), torch.zeros_like(va)
                assert l.cgx_sort_pairs_pingpong(n, end_bit, low, ka.data_ptr(), va.data_ptr(), kb.data_ptr(),
                                                 vb.data_ptr(), ws.data_ptr(), ws.numel(), 0, st) == 0
                torch.cuda.synchronize()
                k, v = (ka, va) if l.cgx_sort_passes(end_bit - (32 - low)) % 2 == 0 else (kb, vb)
                assert torch.equal(v.cpu().long(), want) and torch.equal(k.cpu(), shared[want]), variant
    finally:
        l.cgx_set_sort_variant(-1)
    status = C.c_int(-1)
    assert l.cgx_device_status(C.byref(status), st) == 0 and status.value == 0


def test_plane_map_forward_and_backward(cuda_device):
    """The fused plane-descriptor op against the tensor code it replaces (cgx.synthetic.build_all_map restates the
    reference's caller), differentiated by torch autograd in float64."""
    from cgx.plane_map import plane_map

    g, cam = util.make_case(cfg=2, n=50_000, res=(320, 240))
    dev = cuda_device
    leaves = {k: g[k].to(dev).requires_grad_(True) for k in ("means3D", "scales", "rotations")}
    radii = (torch.arange(50_000, device=dev) % 7 != 0).to(torch.int32)          # some rows skipped
    out = plane_map(leaves["means3D"], leaves["scales"], leaves["rotations"], cam.viewmatrix.to(dev),
                    cam.campos.to(dev), radii)
    gen = torch.Generator().manual_seed(11)
    cot = torch.randn(50_000, 5, generator=gen).to(dev)
    (out * cot).sum().backward()

    ref_leaves = {k: g[k].double().to(dev).requires_grad_(True) for k in ("means3D", "scales", "rotations")}
    ref = _build_all_map_f64(ref_leaves["means3D"], ref_leaves["scales"], ref_leaves["rotations"],
                             cam.viewmatrix.double().to(dev), cam.campos.double().to(dev))
    keep = (radii > 0)[:, None]
    ref = ref * keep
    (ref * cot.double()).sum().backward()

    # float32 forward against float64: unit normals to 1e-5; the distance is a dot product of coordinates of a few
    # hundred metres whose terms cancel, so its float32 rounding is bounded by the coordinates' magnitude
    assert (out[:, :4] - ref[:, :4].float()).abs().max().item() <= 1e-5
    assert (out[:, 4] - ref[:, 4].float()).abs().max().item() <= 1e-6 * 4 * 300.0
    assert not out[radii == 0].any()
    for k in ("means3D", "rotations"):
        a, b = leaves[k].grad.double(), ref_leaves[k].grad
        assert ((a - b).norm() / b.norm()).item() <= 1e-4, k
    assert leaves["scales"].grad is None or not leaves["scales"].grad.any()


def _build_all_map_f64(means3D, scales, rotations, V, campos):
    """gaussian_renderer/__init__.py:1501-1518 in float64 (quaternion [r, x, y, z], row-vector view matrix)."""
    q = torch.nn.functional.normalize(rotations, p=2, dim=-1)
    r, x, y, z = q.unbind(-1)
    two_s = 2.0 / (q * q).sum(-1)
    Rm = torch.stack([1 - two_s * (y * y + z * z), two_s * (x * y - z * r), two_s * (x * z + y * r),
                      two_s * (x * y + z * r), 1 - two_s * (x * x + z * z), two_s * (y * z - x * r),
                      two_s * (x * z - y * r), two_s * (y * z + x * r), 1 - two_s * (x * x + y * y)], -1).view(-1, 3, 3)
    idx = scales.min(dim=-1)[1][..., None, None].expand(-1, 3, -1)
    normal = Rm.gather(2, idx).squeeze(2)
    neg = (normal * (campos - means3D)).sum(-1) < 0.0
    normal = torch.where(neg[:, None], -normal, normal)
    local_normal = normal @ V[:3, :3]
    pts = means3D @ V[:3, :3] + V[3, :3]
    dist = (local_normal * pts).sum(-1).abs()
    return torch.cat([local_normal, torch.ones_like(dist)[:, None], dist[:, None]], 1)


def test_fused_plane_descriptors_equal_the_standalone_op(cuda_device):
    """Batched preprocess with fused plane descriptors == batched preprocess + cgx.plane_map per camera, forward
    and parameter gradients."""
    from cgx.batched import preprocess_gaussians_batched
    from cgx.plane_map import plane_map
    from cgx import runtime as RT

    n, res, B = 40_000, (320, 240), 3
    g, cams = util.S.config(2, n_gaussians=n, n_cameras=B, res=res)
    dev = cuda_device
    settings = RT.TrainingStep(g, cams, dev).settings
    gen = torch.Generator().manual_seed(3)
    cots = [(torch.randn(n, 2, generator=gen).to(dev), torch.randn(n, 4, generator=gen).to(dev),
             torch.randn(n, 5, generator=gen).to(dev)) for _ in range(B)]

    def leaves():
        return {k: g[k].to(dev).requires_grad_(True) for k in ("means3D", "scales", "rotations", "opacities")}

    a = leaves()
    fused = preprocess_gaussians_batched(a["means3D"], a["scales"], a["rotations"], None, a["opacities"], settings,
                                         planes=True)
    loss = sum((t[0] * c[0]).sum() + (t[2] * c[1]).sum() + (t[5] * c[2]).sum() for t, c in zip(fused, cots))
    loss.backward()

    b = leaves()
    plain = preprocess_gaussians_batched(b["means3D"], b["scales"], b["rotations"], None, b["opacities"], settings)
    maps = [plane_map(b["means3D"], b["scales"], b["rotations"], rs.viewmatrix, rs.campos, t[3])
            for rs, t in zip(settings, plain)]
    loss = sum((t[0] * c[0]).sum() + (t[2] * c[1]).sum() + (m * c[2]).sum() for t, m, c in zip(plain, maps, cots))
    loss.backward()

    for t, u, m in zip(fused, plain, maps):
        assert torch.equal(t[3], u[3]) and torch.equal(t[0], u[0]) and torch.equal(t[2], u[2])
        assert torch.allclose(t[5], m, rtol=1e-6, atol=1e-6)
        assert (t[5][t[3] == 0] == 0).all()
    for k in ("means3D", "scales", "rotations", "opacities"):
        ga, gb = a[k].grad, b[k].grad
        assert ((ga - gb).norm() / gb.norm()).item() <= 1e-5, k


def test_prefetched_pair_count_gives_the_same_render(cuda_device):
    """Counting started ahead of render_gaussians (several cameras queued before the first host read) must be picked
    up by identity of the inputs and change nothing; an unrelated call must not pick it up."""
    from diff_gaussian_rasterization import GaussianRasterizer, _C

    dev = cuda_device
    g, cam = util.make_case(cfg=2, n=30_000, res=(320, 240))
    rs = settings_for(cam, dev)
    rast = GaussianRasterizer(rs)
    gd = to_dev(g, dev)
    args = cuda_args()
    m2, _, co, radii, depths = rast.preprocess_gaussians(gd["means3D"], gd["scales"], gd["rotations"], gd["sh"],
                                                         gd["opacities"], args)
    TX, TY = (cam.W + 15) // 16, (cam.H + 15) // 16
    local = torch.ones(TY, TX, dtype=torch.bool, device=dev)
    half = local.clone()
    half[TY // 2:] = False

    def render(loc):
        return _C.render_gaussians(rs.bg, cam.H, cam.W, m2.detach(), depths, radii, co.detach(), gd["rgb"], loc,
                                   rs.viewmatrix, rs.campos, cam.tanfovx, cam.tanfovy, gd["all_map"], True, True, args)

    plain_full, plain_half = render(local), render(half)
    _C.prefetch_num_rendered(cam.H, cam.W, m2.detach(), radii, local)
    _C.prefetch_num_rendered(cam.H, cam.W, m2.detach(), radii, half)
    assert len(_C._PREFETCH) == 2
    pre_half, pre_full = render(half), render(local)          # picked up out of order, by identity
    assert len(_C._PREFETCH) == 0
    for a, b in ((plain_full, pre_full), (plain_half, pre_half)):
        assert a[0] == b[0] and a[0] > 0
        for x, y in zip(a[1:8], b[1:8]):
            assert torch.equal(x, y)
    assert plain_half[0] < plain_full[0]


def test_chunked_batched_preprocess_is_identical(cuda_device):
    """The same two launches split into chunks of Gaussians (the hooks an end-to-end caller uses to overlap its host
    copies): bit-identical outputs and gradients, hooks called once per chunk with the right rows."""
    from cgx.batched import Pipeline, chunk_bounds, preprocess_gaussians_batched
    from cgx import runtime as RT

    n, B = 10_000, 2
    g, cams = util.S.config(2, n_gaussians=n, n_cameras=B, res=(320, 240))
    dev = cuda_device
    settings = RT.TrainingStep(g, cams, dev).settings
    gen = torch.Generator().manual_seed(8)
    cots = [(torch.randn(n, 2, generator=gen).to(dev), torch.randn(n, 4, generator=gen).to(dev),
             torch.randn(n, 5, generator=gen).to(dev)) for _ in range(B)]
    results = []
    for chunks in (1, 3):
        leaves = {k: g[k].to(dev).requires_grad_(True) for k in ("means3D", "scales", "rotations", "opacities")}
        bounds = chunk_bounds(n, chunks)
        seen = []
        ready = []
        for _ in bounds:
            ev = torch.cuda.Event()
            ev.record()
            ready.append(ev)
        pipe = Pipeline(bounds, ready=ready, done=lambda i, lo, hi, grads: seen.append((i, lo, hi, len(grads))))
        out = preprocess_gaussians_batched(leaves["means3D"], leaves["scales"], leaves["rotations"], None,
                                           leaves["opacities"], settings, planes=True, pipeline=pipe)
        sum((t[0] * c[0]).sum() + (t[2] * c[1]).sum() + (t[5] * c[2]).sum() for t, c in zip(out, cots)).backward()
        assert seen == [(i, lo, hi, 4) for i, (lo, hi) in enumerate(bounds)]
        results.append((out, {k: v.grad.clone() for k, v in leaves.items()}))
    assert len(chunk_bounds(n, 3)) == 3
    (a, ga), (b, gb) = results
    for ta, tb in zip(a, b):
        for x, y in zip(ta, tb):
            assert torch.equal(x, y)
    for k in ga:
        assert torch.equal(ga[k], gb[k]), k


def test_end_to_end_steps_follow_their_host_inputs(cuda_device):
    """`TrainingStep.run_e2e` (host parameters and upstream-gradient images in, host gradients out; uploads of one call
    run beside the kernels of the call before it, in alternating device buffers): the gradients that arrive on the
    host are those of a device-resident step on the same inputs, call after call, also when the host inputs change
    between calls that are still in flight."""
    from cgx import runtime as RT

    dev = cuda_device
    g, cams = util.S.config(2, n_gaussians=30_000, n_cameras=3, res=(320, 240))
    names = ("means3D", "scales", "rotations", "opacities")

    def resident(host, cot_host):
        step = RT.TrainingStep(g, cams, dev)
        with torch.no_grad():
            for k in names:
                step.params[k].copy_(host[k])
            for dst, src in zip(step.cot, cot_host):
                for d, s in zip(dst, src):
                    d.copy_(s)
        step.run()
        torch.cuda.synchronize()
        return {k: step.params[k].grad.cpu() for k in names}

    step = RT.TrainingStep(g, cams, dev)
    want = [resident(step.host, step.cot_host)]
    got = []
    for call in range(5):
        if call in (2, 4):                      # new host inputs between groups of back-to-back calls
            step.finish_e2e()                   # the pinned buffers are being read until the uploads have run
            step.host["opacities"].mul_(0.8)
            step.host["means3D"].add_(0.01)
            for cs in step.cot_host:
                cs[0].mul_(-0.5)
            want.append(resident(step.host, step.cot_host))
        step.run_e2e(chunks=3)
        if call in (1, 3, 4):
            step.finish_e2e()
            got.append({k: v.clone() for k, v in step.grad_host.items()})
    assert len(got) == len(want) == 3
    for a, b in zip(got, want):
        for k in names:
            rel = ((a[k] - b[k]).norm() / b[k].norm()).item()
            assert rel <= 1e-5, (k, rel)
    assert ((want[0]["opacities"] - want[1]["opacities"]).norm() / want[0]["opacities"].norm()).item() > 1e-2


def test_camera_streams_do_not_change_the_step(cuda_device):
    """The single-GPU step with its cameras on one, two or three CUDA streams: same radii, same parameter gradients
    (the atomics' order differs, nothing else), repeated so that buffers are reused across steps."""
    from cgx import runtime as RT

    dev = cuda_device
    g, cams = util.S.config(2, n_gaussians=40_000, n_cameras=5, res=(320, 240))
    names = ("means3D", "scales", "rotations", "opacities")
    results = []
    for n_streams in (1, 2, 3):
        step = RT.TrainingStep(g, cams, dev)
        step.render_streams = n_streams
        for _ in range(3):
            step.run()
        torch.cuda.synchronize()
        results.append(({k: step.params[k].grad.clone() for k in names}, [r.clone() for r, _ in step.last]))
    base_grads, base_radii = results[0]
    for grads, radii in results[1:]:
        for a, b in zip(radii, base_radii):
            assert torch.equal(a, b)
        for k in names:
            rel = ((grads[k] - base_grads[k]).norm() / base_grads[k].norm()).item()
            assert rel <= 1e-5, (k, rel)


def test_row_driven_preprocess_backward_equals_dense(cuda_device):
    """cgx_preprocess_bwd_rows (one thread per returned gradient row, sums by atomics) against the camera-batched
    backward over dense per-camera cotangents built from the same rows: several segments per camera, Gaussians with
    two rows for one camera (sent to two ranks), Gaussians with no row at all."""
    import ctypes as C

    from cgx.batched import _cams, _ptrs, preprocess_gaussians_batched
    from cgx.exchange import _RowSegment
    from cgx import runtime as RT
    from diff_gaussian_rasterization import _lib

    n, B = 30_000, 3
    g, cams = util.S.config(2, n_gaussians=n, n_cameras=B, res=(320, 240))
    dev = cuda_device
    settings = RT.TrainingStep(g, cams, dev).settings
    names = ("means3D", "scales", "rotations", "opacities")
    leaves = {k: g[k].to(dev).requires_grad_(True) for k in names}
    out = preprocess_gaussians_batched(leaves["means3D"], leaves["scales"], leaves["rotations"], None,
                                       leaves["opacities"], settings, planes=True)
    gen = torch.Generator().manual_seed(5)
    rows, index, segs, start = [], [], [], 0
    dense = [(torch.zeros(n, 2, device=dev), torch.zeros(n, 4, device=dev), torch.zeros(n, 5, device=dev))
             for _ in range(B)]
    for b in range(B):
        vis = (out[b][3] > 0).nonzero().flatten().cpu()
        pick = vis[torch.rand(len(vis), generator=gen) < 0.7]
        assert len(pick) > 1000
        for part in (pick, pick[::7]):                        # the second segment repeats every seventh Gaussian
            r = torch.randn(len(part), 14, generator=gen).to(dev)
            idx = part.to(dev)
            rows.append(r)
            index.append(idx.to(torch.int32))
            segs.append((start, len(part), b))
            start += len(part)
            dense[b][0].index_add_(0, idx, r[:, 0:2])
            dense[b][1].index_add_(0, idx, r[:, 5:9])
            dense[b][2].index_add_(0, idx, r[:, 9:14])
    segs.insert(2, (start, 0, 1))                             # an empty segment is legal
    sum((t[0] * d[0]).sum() + (t[2] * d[1]).sum() + (t[5] * d[2]).sum() for t, d in zip(out, dense)).backward()
    want = {k: leaves[k].grad for k in names}

    rows, index = torch.cat(rows).contiguous(), torch.cat(index).contiguous()
    arr = (_RowSegment * len(segs))()
    for e, (a, cnt, b) in zip(arr, segs):
        e.start, e.count, e.camera = a, cnt, b
    l = _lib.lib()
    got = {"means3D": torch.empty(n, 3, device=dev), "scales": torch.empty(n, 3, device=dev),
           "rotations": torch.empty(n, 4, device=dev), "opacities": torch.empty(n, 1, device=dev)}
    work = torch.empty(l.cgx_preprocess_bwd_rows_workspace_bytes(n), dtype=torch.uint8, device=dev)
    cam_arr, keep = _cams(settings)
    campos = [rs.campos.contiguous() for rs in settings]
    p = {k: leaves[k].detach().contiguous() for k in names}

    def call(nbytes, ncols=14):
        return l.cgx_preprocess_bwd_rows(
            n, len(segs), arr, ncols, C.c_void_p(rows.data_ptr()), C.c_void_p(index.data_ptr()),
            C.c_void_p(p["means3D"].data_ptr()), C.c_void_p(p["scales"].data_ptr()), 1.0,
            C.c_void_p(p["rotations"].data_ptr()), B, cam_arr, _ptrs(campos), C.c_void_p(work.data_ptr()), nbytes,
            C.c_void_p(got["means3D"].data_ptr()), C.c_void_p(got["scales"].data_ptr()),
            C.c_void_p(got["rotations"].data_ptr()), C.c_void_p(got["opacities"].data_ptr()),
            C.c_void_p(torch.cuda.current_stream().cuda_stream))

    assert call(work.numel() - 1) == _lib.CGX_ENOMEM
    assert call(work.numel(), ncols=12) == _lib.CGX_EINVAL
    assert call(work.numel()) == 0
    torch.cuda.synchronize()
    for k in names:
        rel = ((got[k] - want[k]).norm() / want[k].norm()).item()
        assert rel <= 1e-5, (k, rel)
    untouched = torch.ones(n, dtype=torch.bool, device=dev)
    untouched[index.long()] = False
    assert untouched.any() and (got["means3D"][untouched] == 0).all() and (got["opacities"][untouched] == 0).all()
