"""Plane descriptors (PGSR all_map) against golden vectors made by the reference's own statements
(gaussian_renderer/__init__.py:1501-1518, executed on CPU by tests/golden/make_all_map_golden.py).

cgx.synthetic.build_all_map is the tensor form the GPU tests hold the kernels to (forward values and, through
float64 autograd, gradients); this file holds build_all_map to the reference.  On a GPU the stand-alone kernel is
compared with the same vectors directly."""
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden" / "all_map_1024.npz"


def _load():
    z = np.load(GOLDEN)
    return {k: torch.from_numpy(z[k]) for k in z.files}


def test_tensor_form_equals_the_reference_statements():
    from cgx import synthetic as S

    g = _load()
    for c in range(2):
        cam = SimpleNamespace(campos=g[f"campos{c}"], viewmatrix=g[f"viewmatrix{c}"])
        got = S.build_all_map(g["means3D"], g["scales"], g["rotations"], cam)
        want = g[f"all_map{c}"]
        assert got.shape == want.shape == (1024, 5)
        assert torch.equal(got[:, 3], torch.ones(1024))
        assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
        # the flip towards the camera happened for the same Gaussians (about half of them)
        flipped = g[f"flipped{c}"]
        assert 300 < int(flipped.sum()) < 724
    # the vectors exercise ties of the smallest axis and quaternions of any norm
    assert int((g["scales"][:, 0] == g["scales"][:, 1]).sum()) >= 10
    norms = g["rotations"].norm(dim=1)
    assert float(norms.min()) < 0.2 and float(norms.max()) > 3.0


@pytest.mark.gpu
def test_kernel_equals_the_reference_statements(cuda_device):
    from cgx.plane_map import plane_map

    g = _load()
    dev = cuda_device
    for c in range(2):
        radii = torch.ones(1024, dtype=torch.int32, device=dev)
        got = plane_map(g["means3D"].to(dev), g["scales"].to(dev), g["rotations"].to(dev),
                        g[f"viewmatrix{c}"].to(dev), g[f"campos{c}"].to(dev), radii)
        want = g[f"all_map{c}"].to(dev)
        # the sign of a normal whose dot product with the view direction is within rounding of zero may differ
        # between two float32 evaluations: a handful of rows may disagree, a wrong axis or tie rule would not pass
        assert torch.allclose(got[:, 3], want[:, 3])
        close = torch.isclose(got, want, rtol=1e-4, atol=1e-4).all(dim=1)
        assert int((~close).sum()) <= 5
