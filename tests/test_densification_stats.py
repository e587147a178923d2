"""Densification statistics: dense masked updates equal the reference's boolean-mask updates."""
import torch

import util  # noqa: F401  (puts the package on sys.path)
from cgx.densification import DensificationStats


def test_updates_match_boolean_mask_form():
    gen = torch.Generator().manual_seed(0)
    n = 1000
    stats = DensificationStats(n, "cpu")
    accum = torch.zeros(n, 1)
    denom = torch.zeros(n, 1)
    max_r = torch.zeros(n, dtype=torch.int32)
    for cam in range(3):
        radii = torch.randint(0, 4, (n,), generator=gen, dtype=torch.int32) * (torch.rand(n, generator=gen) > 0.4)
        radii = radii.to(torch.int32)
        m2 = torch.zeros(n, 2, requires_grad=True)
        m2.grad = torch.randn(n, 2, generator=gen)
        stats.update(radii, m2)
        vis = radii > 0                                   # scene/gaussian_model.py:1200-1204 in mask form
        accum[vis] += torch.norm(m2.grad[vis, :2], dim=-1, keepdim=True)
        denom[vis] += 1
        max_r[vis] = torch.max(max_r[vis], radii[vis])
    assert torch.allclose(stats.grad_accum, accum) and torch.equal(stats.denom, denom)
    assert torch.equal(stats.max_radii2D, max_r)
    mean = stats.mean_gradient()
    assert torch.isfinite(mean).all() and (mean[denom == 0] == 0).all()


def test_camera_without_gradient_is_skipped():
    stats = DensificationStats(4, "cpu", track_max_radii=False)
    stats.update(torch.ones(4, dtype=torch.int32), torch.zeros(4, 2, requires_grad=True))
    assert not stats.denom.any() and stats.max_radii2D is None


def test_anchor_statistics_match_the_reference_method():
    """cgx.densification.AnchorStatistics against golden vectors made by the reference's own training_statis body
    (tests/golden/make_statis_golden.py): three calls in a row, accumulators carried over."""
    import numpy as np

    from cgx.densification import AnchorStatistics

    z = np.load(util.GOLDEN / "anchor_statis.npz")
    st = AnchorStatistics(int(z["N"]), int(z["K"]), "cpu")
    for call in range(3):
        t = {k: torch.from_numpy(z[f"{k}{call}"]) for k in ("avm", "opacity", "sel", "upd", "grad")}
        st.training_statis(t["grad"], t["opacity"], t["upd"], t["sel"], t["avm"])
    for name in ("opacity_accum", "anchor_demon", "offset_gradient_accum", "offset_denom"):
        got, want = getattr(st, name), torch.from_numpy(z[name])
        assert torch.allclose(got, want, rtol=1e-6, atol=1e-6), name
    assert float(st.offset_denom.sum()) > 0 and float(st.opacity_accum.sum()) > 0
