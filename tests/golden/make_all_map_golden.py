"""Generate golden vectors for the PGSR plane descriptors by executing the reference's OWN statements
(gaussian_renderer/__init__.py, the block from `rotation_matrices = quaternion_to_matrix(` to
`input_all_map[:, 4] = local_distance`, lines 1501-1518) on seeded CPU inputs:

    python tests/golden/make_all_map_golden.py /path/to/reference [out_dir]

The statements sit in the middle of the reference's render function, so they are cut out of the source text between
those two markers, dedented, and executed with the variables they read.  Two things they need are not in the
reference tree: `.cuda()` (dropped from the text: the vectors are made on CPU) and `quaternion_to_matrix`, which the
reference imports from pytorch3d (pinned `pytorch3d==0.3.0` in its environment.yml, not installed here); it is
restated below from the library's documented formula for real-first quaternions.  The scales go in as the
logarithms the reference's statement expects (it takes `exp` before looking for the smallest axis).
tests/test_all_map_golden.py pins cgx.synthetic.build_all_map (what the kernels are tested against) to the file.
"""
import sys
import textwrap
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def quaternion_to_matrix(q):
    """pytorch3d.transforms.quaternion_to_matrix: real part first, any norm (the result is divided by |q|^2)."""
    r, i, j, k = torch.unbind(q, -1)
    two_s = 2.0 / (q * q).sum(-1)
    o = torch.stack((1 - two_s * (j * j + k * k), two_s * (i * j - k * r), two_s * (i * k + j * r),
                     two_s * (i * j + k * r), 1 - two_s * (i * i + k * k), two_s * (j * k - i * r),
                     two_s * (i * k - j * r), two_s * (j * k + i * r), 1 - two_s * (i * i + j * j)), -1)
    return o.reshape(q.shape[:-1] + (3, 3))


def reference_block(ref):
    src = (ref / "gaussian_renderer" / "__init__.py").read_text()
    first = src.index("rotation_matrices = quaternion_to_matrix(torch.nn.functional.normalize(rotations_redistributed, p=2")
    last_line = "input_all_map[:, 4] = local_distance"
    last = src.index(last_line, first) + len(last_line)
    start = src.rfind("\n", 0, first) + 1
    return textwrap.dedent(src[start:last]).replace(".cuda()", "")


def look_at(eye, target):
    """World-to-camera matrix in the reference's row-vector convention (points are multiplied from the left)."""
    eye, target = torch.tensor(eye), torch.tensor(target)
    z = torch.nn.functional.normalize(target - eye, dim=0)
    x = torch.nn.functional.normalize(torch.linalg.cross(z, torch.tensor([0.0, 0.0, 1.0])), dim=0)
    y = torch.linalg.cross(z, x)
    R = torch.stack([x, y, z], 1)                       # columns: camera axes in world coordinates
    V = torch.eye(4)
    V[:3, :3] = R
    V[3, :3] = -(eye @ R)
    return V, eye


def main():
    ref = Path(sys.argv[1])
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    code = reference_block(ref)
    gen = torch.Generator().manual_seed(1501)
    P = 1024
    xyz = (torch.rand(P, 3, generator=gen) * 2 - 1) * torch.tensor([100.0, 100.0, 15.0])
    log_scales = torch.randn(P, 3, generator=gen) * 0.7 - 1.0
    log_scales[::97, 1] = log_scales[::97, 0]           # ties of the smallest axis: the first one must win
    rotations = torch.randn(P, 4, generator=gen) * torch.rand(P, 1, generator=gen) * 3.0   # any norm
    out = dict(means3D=xyz.numpy(), scales=torch.exp(log_scales).numpy(), rotations=rotations.numpy())
    for c, (eye, target) in enumerate((((0.0, -60.0, 60.0), (0.0, 0.0, 0.0)), ((150.0, 40.0, 25.0), (0.0, 10.0, 5.0)))):
        V, campos = look_at(eye, target)
        ns = dict(torch=torch, quaternion_to_matrix=quaternion_to_matrix, rotations_redistributed=rotations.clone(),
                  scales_redistributed=log_scales.clone(), xyz_redistributed=xyz.clone(),
                  means2D_redistributed=torch.zeros(P, 2), cam_id=0,
                  batched_cameras=[types.SimpleNamespace(camera_center=campos, world_view_transform=V)])
        exec(code, ns)
        out[f"viewmatrix{c}"], out[f"campos{c}"] = V.numpy(), campos.numpy()
        out[f"all_map{c}"] = ns["input_all_map"].numpy()
        out[f"flipped{c}"] = ns["neg_mask"].numpy()
        print(c, "flipped towards the camera:", int(ns["neg_mask"].sum()), "of", P)
    np.savez_compressed(out_dir / "all_map_1024.npz", **out)
    print((out_dir / "all_map_1024.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
