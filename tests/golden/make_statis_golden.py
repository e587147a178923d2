"""Golden vectors for the anchor statistics, made by the reference's OWN method body
(scene/gaussian_model.py ``GaussianModel.training_statis``): the function is cut out of the source file with `ast`
(the module itself needs packages that are not installed here) and run on a stand-in object that holds the four
accumulators:

    python tests/golden/make_statis_golden.py /path/to/reference [out_dir]

Three calls in a row on seeded masks (the accumulators carry over), inputs and final accumulators stored."""
import ast
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def reference_method(ref):
    src = (ref / "scene" / "gaussian_model.py").read_text()
    tree = ast.parse(src)
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "training_statis":
            code = ast.get_source_segment(src, node)
            ns = {"torch": torch}
            exec(compile(ast.parse("import torch\n" + __import__("textwrap").dedent(code)), "training_statis", "exec"), ns)
            return ns["training_statis"]
    raise RuntimeError("training_statis not found")


def main():
    ref = Path(sys.argv[1])
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    fn = reference_method(ref)
    N, K = 500, 10
    gen = torch.Generator().manual_seed(77)
    me = SimpleNamespace(n_offsets=K, opacity_accum=torch.zeros(N, 1), anchor_demon=torch.zeros(N, 1),
                         offset_gradient_accum=torch.zeros(N * K, 1), offset_denom=torch.zeros(N * K, 1))
    out = {"N": np.int64(N), "K": np.int64(K)}
    for call in range(3):
        avm = torch.rand(N, generator=gen) > 0.4
        V = int(avm.sum())
        opacity = torch.randn(V * K, 1, generator=gen)
        sel = torch.rand(V * K, generator=gen) > 0.5
        G = int(sel.sum())
        upd = torch.rand(G, generator=gen) > 0.3
        grad = torch.randn(G, 3, generator=gen)
        fn(me, SimpleNamespace(grad=grad), opacity, upd, sel, avm)
        out.update({f"avm{call}": avm.numpy(), f"opacity{call}": opacity.numpy(), f"sel{call}": sel.numpy(),
                    f"upd{call}": upd.numpy(), f"grad{call}": grad.numpy()})
    out.update(opacity_accum=me.opacity_accum.numpy(), anchor_demon=me.anchor_demon.numpy(),
               offset_gradient_accum=me.offset_gradient_accum.numpy(), offset_denom=me.offset_denom.numpy())
    np.savez_compressed(out_dir / "anchor_statis.npz", **out)
    print((out_dir / "anchor_statis.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
