"""Generate the golden record of the anchor redistribution by running the reference's OWN method
(scene/gaussian_model.py `GaussianModel.all2all_gaussian_state`, lines 1485-1515, applied to every state tensor as
`redistribute_gaussians` :1683-1764 does) on two gloo ranks on CPU:

    python tests/golden/make_redistribute_golden.py /path/to/reference [out_dir]

The method is cut out of the class with `ast` (the module imports pytorch3d, the trainer's utilities and more) and
called with a stand-in for `self` that answers `group_for_redistribution()` with the gloo world group.  The only
change to the source text is the device of the receive buffers ("cuda" -> "cpu"); gloo's missing all_to_all of
unequal lists is answered by all_to_all_single with split sizes (booleans travel as bytes).  The count exchange in
front of it is the reference's (:1718-1735: bincount of the destinations, all-gather).  States and destinations are
those of tests/test_redistribute.py.  Stored: the size table and dtype / shape / SHA-256 of every tensor every rank
ends up with.
"""
import ast
import hashlib
import json
import os
import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
SIZES = (1000, 777)


def reference_method(ref):
    src = (Path(ref) / "scene" / "gaussian_model.py").read_text()
    cls = next(n for n in ast.parse(src).body if isinstance(n, ast.ClassDef) and n.name == "GaussianModel")
    fn = next(n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == "all2all_gaussian_state")
    import textwrap

    return textwrap.dedent(ast.get_source_segment(src, fn, padded=True)).replace('device="cuda"', 'device="cpu"')


def digest(t):
    t = t.detach().contiguous()
    raw = t.view(torch.uint8) if t.dtype == torch.bool else t
    return [str(t.dtype), list(t.shape), hashlib.sha256(raw.numpy().tobytes()).hexdigest()]


def worker(rank, ws, port, code, out_dir):
    for p in (ROOT, ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        import test_redistribute as T

        def all_to_all(outputs, inputs, group=None):
            as_bytes = outputs[0].dtype == torch.bool
            send = torch.cat([t.reshape(t.shape[0], -1) for t in inputs]).contiguous()
            recv = torch.empty(sum(o.shape[0] for o in outputs), send.shape[1], dtype=send.dtype)
            if as_bytes:
                send, recv = send.to(torch.uint8), recv.to(torch.uint8)
            dist.all_to_all_single(recv, send, [o.shape[0] for o in outputs], [t.shape[0] for t in inputs], group=group)
            for o, piece in zip(outputs, recv.split([o.shape[0] for o in outputs])):
                o.copy_(piece.reshape(o.shape).to(o.dtype))

        dist.all_to_all = all_to_all
        ns = {"torch": torch}
        exec(code, ns)
        me = SimpleNamespace(group_for_redistribution=lambda: dist.group.WORLD)
        states, destination = T._states(rank, SIZES[rank])
        # the count exchange of redistribute_gaussians
        local2j_send_size = torch.bincount(destination, minlength=ws).int()
        i2j_send_size = torch.zeros((ws, ws), dtype=torch.int)
        dist.all_gather_into_tensor(i2j_send_size.view(-1), local2j_send_size)     # gloo wants the flat shape
        i2j_send_size = i2j_send_size.cpu().numpy().tolist()
        moved = [ns["all2all_gaussian_state"](me, s, destination, i2j_send_size) for s in states]
        Path(out_dir, f"rank{rank}.json").write_text(json.dumps({"table": i2j_send_size,
                                                                 "out": [digest(t) for t in moved]}))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def main():
    ref = sys.argv[1]
    out_dir = Path(sys.argv[2]) if len(sys.argv) > 2 else HERE
    sys.path.insert(0, str(ROOT / "tests"))
    import test_redistribute as T

    code = reference_method(ref)
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(worker, args=(2, T._free_port(), code, tmp), nprocs=2, join=True)
        ranks = [json.loads(Path(tmp, f"rank{r}.json").read_text()) for r in range(2)]
    (out_dir / "redistribute_golden.json").write_text(json.dumps({"sizes": list(SIZES), "ranks": ranks}))
    print("size table [src][dst]:", ranks[0]["table"], "rows per rank afterwards:", [r["out"][0][1][0] for r in ranks])
    print((out_dir / "redistribute_golden.json").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
