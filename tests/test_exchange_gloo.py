"""World-size-2 gloo runs of the Gaussian all-to-all on CPU (benchmark configuration 0: 50k Gaussians, two
256x144 cameras).  Checks the ordering contract, that the concatenation of both ranks' renders equals the
single-process render, and that gradients flow back through the reverse exchange to the owning rank."""
import os
import socket
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
N_GAUSS = 6000
RES = (128, 160)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _scene():
    import util

    g, cams = util.S.config(0, n_gaussians=N_GAUSS, res=RES)
    return g, cams


def _preprocess_local(g, cam, sel):
    from oracle import cpu_raster as O

    m2, dep, rad, cov3, co = O.preprocess_fwd(g["means3D"][sel], g["scales"][sel], g["rotations"][sel],
                                              g["opacities"][sel], cam.viewmatrix, cam.projmatrix, cam.W, cam.H,
                                              cam.tanfovx, cam.tanfovy)
    return m2, dep, rad, co


def _worker(rank, ws, port, out_dir):
    for p in (ROOT, ROOT / "citygs-x_b200", ROOT / "tests"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        import util
        from oracle.exchange_backend import OracleBackend
        from cgx import exchange
        from cgx import workload_division as WD
        from oracle import cpu_raster as O

        g, cams = _scene()
        ctx = WD.DivisionContext(image_height=cams[0].H, image_width=cams[0].W, rank=rank, world_size=ws,
                                 bsz=len(cams), device="cpu")
        hist = WD.DivisionStrategyHistoryFinal(cams, ws, rank, ctx=ctx)
        # skew the heuristic so that the cut falls inside camera 0 (both ranks render part of it)
        hist.accum_heuristic[cams[0].uid] = torch.ones(ctx.tile_y) * 3.0
        strategies, tasks = WD.start_strategy_final(cams, hist, ctx=ctx)
        sel = slice(rank, None, ws)
        screen, leaves = [], []
        for cam in cams:
            m2, dep, rad, co = _preprocess_local(g, cam, sel)
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
        out = exchange.all_to_all_communication_final(rasts, screen, args, strategies, backend=OracleBackend(),
                                                      piggyback=[rank + 0.25, -1.0, 3.5e-3])
        m2r, rgbr, cor, radr, depr, m3r, scr, rotr, sizes, sent, send_index, stats = out

        result = {"sizes": sizes, "strategies": [(s.gpu_ids, s.division_pos) for s in strategies], "renders": {}}
        # every received tensor of every camera, as the reference returns them (for the golden comparison)
        result["received_all"] = [[t[k].detach().clone() for t in (m2r, rgbr, cor, radr, depr, m3r, scr, rotr)]
                                  for k in range(len(cams))]
        heads = []
        for k, cam in enumerate(cams):
            local = strategies[k].get_compute_locally()
            # a weighted sum of everything received, so that every received row gets a distinct gradient
            w = torch.arange(1, m2r[k].shape[0] + 1, dtype=torch.float32)[:, None] / 100.0
            heads.append((m2r[k] * w).sum() + (rgbr[k] * w * 2).sum() + (cor[k] * w * 3).sum()
                         + (m3r[k] * w * 4).sum() + (scr[k] * w * 5).sum() + (rotr[k] * w * 6).sum())
            if local is None:
                continue
            am = util.S.build_all_map(m3r[k].detach(), scr[k].detach(), rotr[k].detach(), cam)
            b = O.bin_and_sort(m2r[k].detach(), depr[k], radr[k], local, cam.W, cam.H)
            f = O.render_fwd(m2r[k].detach(), cor[k].detach(), rgbr[k].detach(), am, b["ranges"], b["point_list"],
                             local, torch.zeros(3), cam.W, cam.H, cam.tanfovx, cam.tanfovy)
            result["renders"][k] = dict(color=f["color"], all_map=f["out_all_map"], local=local,
                                        n=m2r[k].shape[0])
            result.setdefault("received", {})[k] = dict(m2=m2r[k].detach().clone(), rad=radr[k].clone(),
                                                        dep=depr[k].clone(), m3=m3r[k].detach().clone())
        torch.stack(heads).sum().backward()
        result["grads"] = [[t.grad.clone() if t.grad is not None else None for t in lv] for lv in leaves]
        result["stats"] = stats
        torch.save(result, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.fixture(scope="module")
def two_rank_run(tmp_path_factory):
    out = tmp_path_factory.mktemp("gloo")
    for attempt in range(2):              # the rendezvous port can be taken between its choice and its use: once more
        try:
            mp.spawn(_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
            break
        except Exception:
            if attempt:
                raise
    return [torch.load(out / f"rank{r}.pt", weights_only=False) for r in range(2)]


def test_sizes_and_strategies_agree(two_rank_run):
    r0, r1 = two_rank_run
    assert r0["sizes"] == r1["sizes"]
    assert r0["strategies"] == r1["strategies"]
    # camera 0 is split between both ranks, camera 1 belongs to rank 1 alone
    assert r0["strategies"][0][0] == [0, 1] and r0["strategies"][1][0] == [1]
    sizes = r0["sizes"]          # [src][dst][cam]
    assert sizes[0][0][1] == 0 and sizes[1][0][1] == 0        # nobody sends camera-1 rows to rank 0
    assert r0["stats"]["rows_sent"] == sum(sizes[0][j][k] for j in range(2) for k in range(2))
    assert r0["stats"]["rows_received"] == sum(sizes[i][0][k] for i in range(2) for k in range(2))


def test_piggybacked_floats_reach_every_rank(two_rank_run):
    """Values riding on the size-table all-gather (the balancer's render times) come back bit-exact, per rank."""
    import numpy as np

    want = [[float(np.float32(v)) for v in (r + 0.25, -1.0, 3.5e-3)] for r in range(2)]
    for r in two_rank_run:
        assert r["stats"]["piggyback"] == want


def test_row_order_is_source_major_then_local_index(two_rank_run):
    """Received rows of a camera: all rows of source 0 (ascending local index), then source 1."""
    import util
    from oracle import cpu_raster as O

    g, cams = _scene()
    ctxs = two_rank_run[0]["strategies"]
    for me in range(2):
        for k, cam in enumerate(cams):
            if k not in two_rank_run[me].get("received", {}):
                continue
            gpu_ids, division_pos = ctxs[k]
            j = gpu_ids.index(me)
            bounds = torch.tensor(division_pos, dtype=torch.int32) * ((cam.W + 15) // 16)
            expect_m2, expect_m3 = [], []
            for src in range(2):
                sel = slice(src, None, 2)
                m2, dep, rad, co = _preprocess_local(g, cam, sel)
                mask = O.local2j_mask(m2, rad, bounds, cam.W, cam.H)[:, j]
                expect_m2.append(m2[mask])
                expect_m3.append(g["means3D"][sel][mask])
            got = two_rank_run[me]["received"][k]
            assert torch.equal(got["m2"], torch.cat(expect_m2))
            assert torch.equal(got["m3"], torch.cat(expect_m3))
            assert got["rad"].dtype == torch.int32 and (got["rad"] > 0).all()


def test_union_of_rank_renders_equals_single_process_render(two_rank_run):
    import util
    from oracle import cpu_raster as O

    g, cams = _scene()
    for k, cam in enumerate(cams):
        gg = dict(g)
        gg["rgb"] = util.S.colours_for(g, cam)
        gg["all_map"] = util.S.build_all_map(g["means3D"], g["scales"], g["rotations"], cam)
        full = O.full_step(gg, util.cam_dict(cam))
        color = torch.zeros_like(full["color"])
        covered = torch.zeros(cam.H, cam.W, dtype=torch.bool)
        for r in two_rank_run:
            if k in r["renders"]:
                rr = r["renders"][k]
                m = rr["local"].repeat_interleave(16, 0).repeat_interleave(16, 1)[: cam.H, : cam.W]
                assert not (covered & m).any()
                covered |= m
                color += rr["color"]
        assert covered.all()
        # Gaussians reach a rank in a different order than in the single-process list, so equal-depth ties may
        # blend in another order: compare at tolerance
        assert (color - full["color"]).abs().max().item() < 1e-5


def test_gradients_return_to_the_owner(two_rank_run):
    """Backward through the reverse all-to-all: each owner row receives the sum over the destinations it was sent
    to of that destination's per-row weight."""
    import util
    from oracle import cpu_raster as O

    g, cams = _scene()
    strategies = two_rank_run[0]["strategies"]
    sizes = two_rank_run[0]["sizes"]
    for src in range(2):
        sel = slice(src, None, 2)
        for k, cam in enumerate(cams):
            gpu_ids, division_pos = strategies[k]
            bounds = torch.tensor(division_pos, dtype=torch.int32) * ((cam.W + 15) // 16)
            m2, dep, rad, co = _preprocess_local(g, cam, sel)
            mask = O.local2j_mask(m2, rad, bounds, cam.W, cam.H)
            expect = torch.zeros(m2.shape[0])
            for j, dst in enumerate(gpu_ids):
                idx = mask[:, j].nonzero().flatten()
                # position of these rows in dst's per-camera array: after the rows of lower source ranks
                base = sum(sizes[i][dst][k] for i in range(src))
                expect[idx] += (base + torch.arange(1, idx.numel() + 1)).float() / 100.0
            got = two_rank_run[src]["grads"][k]
            assert torch.allclose(got[0][:, 0], expect, atol=1e-5)            # means2D
            assert torch.allclose(got[1][:, 0], expect * 2, atol=1e-5)        # rgb
            assert torch.allclose(got[2][:, 3], expect * 3, atol=1e-5)        # conic_opacity
            assert torch.allclose(got[3][:, 2], expect * 4, atol=1e-5)        # means3D
            assert torch.allclose(got[4][:, 1], expect * 5, atol=1e-5)        # scales
            assert torch.allclose(got[5][:, 0], expect * 6, atol=1e-5)        # rotations


def test_cuda_backend_refuses_cpu_tensors():
    from cgx import exchange

    b = exchange.CudaPackBackend()
    with pytest.raises(RuntimeError, match="CUDA"):
        b.count(torch.zeros(4, 2), torch.zeros(4, dtype=torch.int32), torch.tensor([0, 4], dtype=torch.int32), 16, 16,
                False, torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.uint8))


def test_p2p_layout_is_consistent_across_ranks():
    """The arena layout of the peer-to-peer transport, computed independently by every rank from the same size
    table, must tile each destination tensor without gaps or overlaps, and the gradient rows every receiver
    returns must land exactly on the sender's send order."""
    import numpy as np
    from cgx import exchange as EX

    rng = np.random.default_rng(3)
    ws, bsz = 5, 3
    S = rng.integers(0, 400, size=(ws, ws, bsz))
    S[:, 2, 1] = 0                         # a camera rank 2 takes no part in
    S[3] = 0                               # a rank that sends nothing
    for fields in (EX._CAM_FIELDS, EX._CAM_FIELDS_PLANES):
        lays = [EX.p2p_layout(S, me, fields) for me in range(ws)]
        widths = [w for _, w in fields]
        for a in lays[1:]:                 # rank-independent parts agree
            for key in ("n_recv", "cam_base", "field_off"):
                assert np.array_equal(a[key], lays[0][key])
            assert a["recv_bytes"] == lays[0]["recv_bytes"] and a["grad_rows_max"] == lays[0]["grad_rows_max"]
        L = lays[0]
        for j in range(ws):
            spans = []
            for k in range(bsz):
                # the sources' row ranges tile [0, n_recv) in source order
                cur = 0
                for i in range(ws):
                    assert lays[i]["first_row"][j, k] == cur
                    cur += S[i, j, k]
                assert cur == L["n_recv"][j, k]
                for f, w in enumerate(widths):
                    lo = L["cam_base"][j, k] + L["field_off"][j, k, f]
                    assert lo % 256 == 0
                    spans.append((lo, lo + L["n_recv"][j, k] * w))
            spans.sort()
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 <= b0                                      # tensors of one arena never overlap
            assert spans[-1][1] <= L["recv_bytes"]
        # gradient rows: receiver `me` returns segment (src i, camera k) to row grad_row[i, k] of i's staging buffer,
        # which must be where i's own send order (destination major, camera minor) put those rows
        for i in range(ws):
            order = np.cumsum(S[i].reshape(-1)) - S[i].reshape(-1)
            for me in range(ws):
                for k in range(bsz):
                    assert lays[me]["grad_row"][i, k] == order[me * bsz + k]
            assert S[i].sum() <= L["grad_rows_max"]


def test_store_order_and_destination_rows_of_the_pack_launch():
    """Host side of the peer-to-peer pack launch: every rank works through the cameras starting with those the rank
    after it renders (no two ranks store into the same peer at the same time while each rank renders the same number
    of cameras), and the destination rows built for all (camera, rank) pairs at once equal the per-camera tables."""
    import numpy as np
    from types import SimpleNamespace as NS
    from cgx import exchange as EX

    ws, bsz = 4, 8
    strategies = [NS(gpu_ids=[k // 2]) for k in range(bsz)]            # two whole cameras per rank
    orders = [EX._camera_order(strategies, me, ws) for me in range(ws)]
    for me, order in enumerate(orders):
        assert sorted(order) == list(range(bsz))
        assert [strategies[k].gpu_ids[0] for k in order[-2:]] == [me, me]          # its own cameras last
    for slot in range(bsz):                                                          # at any time: four different peers
        assert len({strategies[orders[me][slot]].gpu_ids[0] for me in range(ws)}) == ws
    # a camera cut between ranks 1 and 2 is ordered by its first rank
    cut = [NS(gpu_ids=[0]), NS(gpu_ids=[1, 2]), NS(gpu_ids=[3])]
    assert EX._camera_order(cut, 0, ws) == [1, 2, 0]
    assert EX._camera_order(cut, 2, ws) == [2, 0, 1]

    rng = np.random.default_rng(9)
    S = rng.integers(1, 300, size=(ws, ws, 3))
    for planes, fields in ((True, EX._CAM_FIELDS_PLANES), (False, EX._CAM_FIELDS)):
        lay = EX.p2p_layout(S, 1, fields)
        peer_base = np.arange(ws, dtype=np.int64) * (1 << 32) + 4096
        field_ptr = peer_base[:, None, None] + lay["cam_base"][:, :, None] + lay["field_off"]
        order = EX._camera_order(cut, 1, ws)
        ids = [cut[k].gpu_ids for k in order]
        cam = np.repeat(np.asarray(order, dtype=np.int64), [len(i) for i in ids])
        dst = np.concatenate([np.asarray(i, dtype=np.int64) for i in ids])
        rows = EX._destination_rows(field_ptr, lay["first_row"], cam, dst, planes)
        at = 0
        for k in order:                                                # the per-camera construction
            for j in cut[k].gpu_ids:
                want = np.zeros(10, dtype=np.uint64)
                if planes:
                    want[[0, 1, 2, 9, 6, 7]] = field_ptr[j, k, :]
                else:
                    want[:8] = field_ptr[j, k, :]
                want[8] = lay["first_row"][j, k]
                assert np.array_equal(rows[at], want)
                at += 1
        assert at == rows.shape[0] == 4


def _digest(t):
    import hashlib

    t = t.detach().contiguous()
    return [str(t.dtype), list(t.shape), hashlib.sha256(t.numpy().tobytes()).hexdigest()]


def test_exchange_equals_the_reference_function(two_rank_run):
    """tests/golden/exchange_golden.json: digests of what the reference's OWN all_to_all_communication_final
    (gaussian_renderer/__init__.py:596-786, run on two gloo ranks by tests/golden/make_exchange_golden.py on this same
    scene, strategies and loss) returned and back-propagated.  The exchange moves rows and adds gradient rows that
    meet at their owner: every tensor must agree bit for bit."""
    import json

    golden = json.loads((ROOT / "tests" / "golden" / "exchange_golden.json").read_text())
    assert golden["n_gaussians"] == N_GAUSS and golden["res"] == list(RES)
    for rank, run in enumerate(two_rank_run):
        want = golden["ranks"][rank]
        assert run["sizes"] == want["sizes"]
        for k, tensors in enumerate(run["received_all"]):
            for name, t, w in zip(("means2D", "rgb", "conic_opacity", "radii", "depths", "means3D", "scales", "rotations"),
                                  tensors, want["received"][k]):
                assert _digest(t) == w, (rank, k, name)
        for k, grads in enumerate(run["grads"]):
            for name, gt, w in zip(("means2D", "rgb", "conic_opacity", "means3D", "scales", "rotations"), grads,
                                   want["grads"][k]):
                assert _digest(gt) == w, (rank, k, name)
    assert sum(w[1][0] for r in golden["ranks"] for cam in r["received"] for w in cam[:1]) > 1000



def test_prepared_pack_launch_passes_the_same_tables(monkeypatch):
    """The pack launch prepared while the size table is in flight (static part first, destination rows of all
    cameras at once afterwards) must hand the library the same camera table and destination rows as the launch built
    camera by camera.  Host code only: the library call is intercepted, the tensors are CPU stand-ins."""
    import ctypes as C

    import numpy as np
    from cgx import exchange as EX
    from diff_gaussian_rasterization import _C

    seen = []

    def capture(name, fn, n, table_ptr, send_index_ptr, stream, **kw):
        table = np.ctypeslib.as_array(C.cast(table_ptr, C.POINTER(C.c_uint64)), shape=(n, 19)).copy()
        rows = []
        for row in table:
            ws = int(row[3])
            dst = np.ctypeslib.as_array(C.cast(int(row[14]), C.POINTER(C.c_uint64)), shape=(ws, 10)).copy()
            offs = np.ctypeslib.as_array(C.cast(int(row[15]), C.POINTER(C.c_int64)), shape=(ws,)).copy()
            rows.append((dst, offs))
        seen.append((name, table, rows))

    monkeypatch.setattr(_C, "_call", capture)
    monkeypatch.setattr(EX.CudaPackBackend, "_st", staticmethod(lambda: None))
    be = EX.CudaPackBackend()
    gen = torch.Generator().manual_seed(2)
    P, ids = 50, [[0], [1, 2], [3]]
    cams = []
    for k, i in enumerate(ids):
        params = (torch.rand(P, 2, generator=gen), torch.rand(P, 3, generator=gen), torch.rand(P, 4, generator=gen),
                  torch.ones(P, dtype=torch.int32), torch.rand(P, generator=gen), torch.rand(P, 5, generator=gen))
        cams.append(dict(params=params, bounds=torch.arange(len(i) + 1, dtype=torch.int32) * 10, H=160 + k, W=128,
                         avoid=bool(k & 1), workspace=torch.zeros(64, dtype=torch.uint8)))
    order = [1, 2, 0]
    rng = np.random.default_rng(4)
    dst_tables = [rng.integers(1, 1 << 40, size=(len(i), 10)).astype(np.uint64) for i in ids]
    row_offsets = [rng.integers(0, 1000, size=(len(i),)).astype(np.int64) for i in ids]
    send_index = torch.zeros(10, dtype=torch.int32)
    # camera by camera
    be.pack_p2p_batched([dict(cams[k], dst_table=dst_tables[k], row_offsets=row_offsets[k]) for k in order], send_index)
    # prepared
    prep = be.prepare_pack_p2p(cams, order)
    be.pack_p2p_prepared(prep, np.concatenate([dst_tables[k] for k in order]),
                         np.concatenate([row_offsets[k] for k in order]), send_index)
    (name_a, table_a, rows_a), (name_b, table_b, rows_b) = seen
    assert name_a == name_b == "cgx_local2j_pack_p2p_batched"
    keep = [c for c in range(19) if c not in (14, 15)]           # 14 / 15 are the addresses of the two side arrays
    assert np.array_equal(table_a[:, keep], table_b[:, keep])
    assert [int(r[3]) for r in table_b] == [len(ids[k]) for k in order]
    for (dst_a, offs_a), (dst_b, offs_b) in zip(rows_a, rows_b):
        assert np.array_equal(dst_a, dst_b) and np.array_equal(offs_a, offs_b)
