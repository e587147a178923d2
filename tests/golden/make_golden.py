"""Generate golden vectors from the reference's own CUDA rasterizer.

Run on a machine with a CUDA GPU and the reference extension built by oracle/build_ref.py:

    python tests/golden/make_golden.py [out_dir]

For each (small, seeded) case it drives the reference extension's raw entry points on the synthetic scene and
stores every stage's output (preprocess, sorted keys / point list / ranges, images, gradients) as a compressed
.npz.  The CPU tests pin the oracle against these files; the GPU tests compare the CUDA path with them too.
"""
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
for p in (ROOT, ROOT / "citygs-x_b200", ROOT / "tests"):
    sys.path.insert(0, str(p))

CASES = {
    "cfg1_8k_256x144": dict(cfg=1, n=8000, res=(256, 144)),
    "cfg0_6k_200x120_big": dict(cfg=0, n=6000, res=(200, 120), big_scales=True),
}


def main():
    import util
    from oracle import build_ref
    from test_parity_gpu import run_reference

    ref = build_ref.load()
    if ref is None:
        raise SystemExit("reference extension not built: run oracle/build_ref.py where the reference sources are")
    out_dir = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE
    out_dir.mkdir(parents=True, exist_ok=True)
    dev = torch.device("cuda:0")
    for name, case in CASES.items():
        g, cam = util.make_case(**case)
        cot = util.cotangents(cam)
        r = run_reference(ref, g, cam, dev, cot=cot)
        arrays = {k: v.numpy() for k, v in r.items() if isinstance(v, torch.Tensor)}
        arrays["R"] = np.int64(r["R"])
        arrays["case_cfg"] = np.int64(case["cfg"])
        arrays["case_n"] = np.int64(case["n"])
        arrays["case_res"] = np.array(case["res"], dtype=np.int64)
        arrays["case_big"] = np.int64(1 if case.get("big_scales") else 0)
        np.savez_compressed(out_dir / f"{name}.npz", **arrays)
        print(name, "R =", r["R"], "visible =", int((r["radii"] > 0).sum()))


if __name__ == "__main__":
    main()
