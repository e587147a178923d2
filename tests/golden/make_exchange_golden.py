"""Generate the golden record of the Gaussian all-to-all by running the reference's OWN function
(gaussian_renderer/__init__.py `all_to_all_communication_final`, lines 596-786) on two gloo ranks on CPU:

    python tests/golden/make_exchange_golden.py /path/to/reference [out_dir]

The function is cut out of the reference's source with `ast` (the module itself imports the trainer, the scene and
the CUDA extension) and executed with stand-ins for what it reads: `utils.DEFAULT_GROUP` is the gloo world group,
`dist_func` is torch.distributed.nn.functional, and every strategy's `get_local2j_ids` (upstream a CUDA kernel) is
answered by the CPU oracle's band mask, which the GPU tests hold bit for bit to that kernel.  The only change to the
source text is the device of the tensors it creates ("cuda" -> "cpu").  Underneath the function, gloo lacks what
NCCL gives it (all_to_all of unequal lists, byte-counting shape checks): those calls are answered by
all_to_all_single with split sizes and by views, see the worker.  Scene, strategies, inputs and the loss are
those of tests/test_exchange_gloo.py (imported from there), so that test's own run can be compared with this record.
Stored: the size table and, per rank and camera, dtype / shape / SHA-256 of every received tensor and of every
input's gradient (the exchange only moves rows and adds gradient rows: results are exact).
"""
import ast
import json
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def reference_function(ref):
    src = (Path(ref) / "gaussian_renderer" / "__init__.py").read_text()
    node = next(n for n in ast.parse(src).body
                if isinstance(n, ast.FunctionDef) and n.name == "all_to_all_communication_final")
    return ast.get_source_segment(src, node).replace('device="cuda"', 'device="cpu"')


class OracleStrategy:
    """What the reference's function needs of a strategy: gpu_ids and the per-rank index lists of its mask kernel."""

    def __init__(self, strategy, cam):
        self.gpu_ids = strategy.gpu_ids
        self.bounds = torch.tensor(strategy.division_pos, dtype=torch.int32) * ((cam.W + 15) // 16)
        self.cam = cam

    def get_local2j_ids(self, means2D, radii, raster_settings, cuda_args):
        from oracle import cpu_raster as O

        mask = O.local2j_mask(means2D.detach(), radii, self.bounds, self.cam.W, self.cam.H,
                              cuda_args["avoid_pixel_all2all"])
        return [mask[:, rk].nonzero() for rk in range(len(self.gpu_ids))], mask


def worker(rank, ws, port, code, out_dir):
    for p in (ROOT, ROOT / "citygs-x_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        import test_exchange_gloo as T
        import util
        from cgx import workload_division as WD
        import torch.distributed.nn.functional as dist_func

        g, cams = T._scene()
        ctx = WD.DivisionContext(image_height=cams[0].H, image_width=cams[0].W, rank=rank, world_size=ws,
                                 bsz=len(cams), device="cpu")
        hist = WD.DivisionStrategyHistoryFinal(cams, ws, rank, ctx=ctx)
        hist.accum_heuristic[cams[0].uid] = torch.ones(ctx.tile_y) * 3.0
        strategies, _ = WD.start_strategy_final(cams, hist, ctx=ctx)
        sel = slice(rank, None, ws)
        screen, leaves = [], []
        for cam in cams:
            m2, dep, rad, co = T._preprocess_local(g, cam, sel)
            rgb = util.S.colours_for({k: v[sel] for k, v in g.items()}, cam)
            m2.requires_grad_(True)
            co.requires_grad_(True)
            rgb.requires_grad_(True)
            m3 = g["means3D"][sel].clone().requires_grad_(True)
            sc = g["scales"][sel].clone().requires_grad_(True)
            rot = g["rotations"][sel].clone().requires_grad_(True)
            screen.append((m2, rgb, co, rad, dep, m3, sc, rot))
            leaves.append((m2, rgb, co, m3, sc, rot))
        rasts = [SimpleNamespace(raster_settings=SimpleNamespace(image_height=c.H, image_width=c.W)) for c in cams]
        args = [{"avoid_pixel_all2all": False} for _ in cams]
        # NCCL's all_gather_into_tensor takes any output of world_size x the input's bytes (the reference passes
        # (ws, ws, cameras) for a (ws, cameras) input); gloo insists on a (ws * rows, cameras) shape: same bytes
        gather = dist.all_gather_into_tensor

        def flat_gather(output_tensor, input_tensor, group=None):
            return gather(output_tensor.view(-1, *input_tensor.shape[1:]), input_tensor, group=group)

        dist.all_gather_into_tensor = flat_gather
        # The reference exchanges lists of unequal tensors with all_to_all (plain, and the autograd-aware one of
        # torch.distributed.nn.functional).  Gloo has neither for unequal sizes, so both are answered here by
        # all_to_all_single with split sizes: the same rows go to the same ranks.  The rows the reference sends are
        # (n, 1, width) (it indexes with the (n, 1) output of nonzero()) for receive buffers of (n, width): NCCL
        # only counts bytes, here they are reshaped.
        def exchange_lists(outputs, inputs, group):
            width = outputs[0].shape[1:]
            send = torch.cat([t.reshape(-1, *width) for t in inputs]).contiguous()
            recv = torch.empty(sum(o.shape[0] for o in outputs), *width, dtype=send.dtype)
            dist.all_to_all_single(recv, send, [o.shape[0] for o in outputs], [t.shape[0] for t in inputs], group=group)
            return recv

        def plain_all_to_all(output_tensor_list, input_tensor_list, group=None):
            recv = exchange_lists(output_tensor_list, input_tensor_list, group)
            for o, piece in zip(output_tensor_list, recv.split([o.shape[0] for o in output_tensor_list])):
                o.copy_(piece)

        class _AllToAll(torch.autograd.Function):
            @staticmethod
            def forward(ctx, group, n_out, *tensors):
                outputs, inputs = tensors[:n_out], tensors[n_out:]
                ctx.group, ctx.in_rows = group, [t.shape[0] for t in inputs]
                ctx.in_shapes = [t.shape for t in inputs]
                recv = exchange_lists(outputs, [t.detach() for t in inputs], group)
                return tuple(recv.split([o.shape[0] for o in outputs]))

            @staticmethod
            def backward(ctx, *grads):
                width = grads[0].shape[1:]
                back = [torch.empty(n, *width) for n in ctx.in_rows]
                recv = exchange_lists(back, [g.contiguous() for g in grads], ctx.group)
                pieces = recv.split(ctx.in_rows)
                return (None, None) + (None,) * len(grads) + tuple(p.reshape(s) for p, s in zip(pieces, ctx.in_shapes))

        def functional_all_to_all(output_tensor_list, input_tensor_list, group=None):
            outs = _AllToAll.apply(group, len(output_tensor_list), *output_tensor_list, *input_tensor_list)
            for i, o in enumerate(outs):       # the reference reads the results out of the list it passed in
                output_tensor_list[i] = o

        dist.all_to_all = plain_all_to_all
        dist_func = SimpleNamespace(all_to_all=functional_all_to_all)
        ns = {"torch": torch, "dist_func": dist_func, "utils": SimpleNamespace(DEFAULT_GROUP=dist.group.WORLD)}
        exec(code, ns)
        out = ns["all_to_all_communication_final"](rasts, screen, args,
                                                   [OracleStrategy(s, c) for s, c in zip(strategies, cams)])
        m2r, rgbr, cor, radr, depr, m3r, scr, rotr, sizes, _ = out
        heads = []
        for k in range(len(cams)):
            w = torch.arange(1, m2r[k].shape[0] + 1, dtype=torch.float32)[:, None] / 100.0
            heads.append((m2r[k] * w).sum() + (rgbr[k] * w * 2).sum() + (cor[k] * w * 3).sum()
                         + (m3r[k] * w * 4).sum() + (scr[k] * w * 5).sum() + (rotr[k] * w * 6).sum())
        torch.stack(heads).sum().backward()
        rec = {"sizes": sizes,
               "received": [[T._digest(t[k]) for t in (m2r, rgbr, cor, radr, depr, m3r, scr, rotr)]
                            for k in range(len(cams))],
               "grads": [[T._digest(t.grad if t.grad is not None else torch.zeros_like(t)) for t in lv] for lv in leaves]}
        Path(out_dir, f"rank{rank}.json").write_text(json.dumps(rec))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def main():
    ref = sys.argv[1]
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    sys.path.insert(0, str(ROOT / "tests"))
    sys.path.insert(0, str(ROOT / "citygs-x_b200"))
    sys.path.insert(0, str(ROOT))
    import tempfile

    import test_exchange_gloo as T

    code = reference_function(ref)
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(worker, args=(2, T._free_port(), code, tmp), nprocs=2, join=True)
        ranks = [json.loads(Path(tmp, f"rank{r}.json").read_text()) for r in range(2)]
    out = {"n_gaussians": T.N_GAUSS, "res": list(T.RES), "ranks": ranks}
    (out_dir / "exchange_golden.json").write_text(json.dumps(out))
    print("size table [src][dst][cam]:", ranks[0]["sizes"])
    print((out_dir / "exchange_golden.json").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
