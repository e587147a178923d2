"""The CUDA path against the committed golden vectors of the reference's CUDA rasterizer (tests/golden/*.npz)."""
import numpy as np
import pytest
import torch

import util
from test_parity_gpu import FWD_TOL, GRAD_TOL, GRADS, run_ours

pytestmark = pytest.mark.gpu

GOLDEN_FILES = sorted(util.GOLDEN.glob("cfg*.npz"))     # rasterizer cases (the loss cases are loss_*.npz)


@pytest.mark.parametrize("path", GOLDEN_FILES, ids=lambda p: p.stem)
def test_cuda_path_against_golden(path, cuda_device):
    z = np.load(path)
    t = {k: torch.from_numpy(z[k]) for k in z.files}
    g, cam = util.make_case(cfg=int(t["case_cfg"]), n=int(t["case_n"]), res=tuple(int(x) for x in t["case_res"]),
                            big_scales=bool(int(t["case_big"])))
    ours = run_ours(g, cam, cuda_device, cot=util.cotangents(cam))
    for k in ("radii", "means2D", "depths", "conic_opacity", "keys", "point_list", "ranges", "n_contrib_px",
              "n_contrib2loss_px", "n_render", "n_consider", "n_contrib", "out_observe"):
        assert torch.equal(ours[k], t[k]), k
    assert ours["R"] == int(t["R"])
    for k in ("color", "out_all_map", "final_T"):
        assert (ours[k] - t[k]).abs().max().item() <= FWD_TOL, k
    for k in GRADS:
        assert util.rel_l2(ours[k], t[k]) <= GRAD_TOL, (k, util.rel_l2(ours[k], t[k]))


def test_golden_files_present():
    assert len(GOLDEN_FILES) >= 1, "run tests/golden/make_golden.py on a GPU box and commit the .npz files"
