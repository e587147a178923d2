"""The exchange kernels on ONE GPU: the destination "ranks" are separate buffers of the same device, so selection,
counting, packing (send-buffer form, direct-store form, per camera and batched) and the gradient transport can be
checked against the CPU oracle's band mask without a second GPU.  Everything here is data movement: bit-exact."""
import numpy as np
import pytest
import torch

import util
from oracle import cpu_raster as O

pytestmark = pytest.mark.gpu

W, H = 320, 192            # 20 x 12 tiles
BOUNDS_ROWS = [0, 4, 7, 12]  # three bands of tile rows
N = 30_000


def _screen_state(cam_idx, dev):
    g, cam = util.make_case(cfg=2, n=N, res=(W, H), cam_idx=cam_idx)
    pre = O.preprocess_fwd(g["means3D"], g["scales"], g["rotations"], g["opacities"], cam.viewmatrix, cam.projmatrix,
                           cam.W, cam.H, cam.tanfovx, cam.tanfovy)
    means2D, depths, radii, _, conic_opacity = pre
    cpu = (means2D, g["rgb"], conic_opacity, radii, depths, g["means3D"], g["scales"], g["rotations"])
    return cpu, tuple(t.to(dev).contiguous() for t in cpu)


def _expected_rows(cpu, bounds):
    mask = O.local2j_mask(cpu[0], cpu[3], bounds, W, H)
    return [mask[:, j].nonzero().flatten() for j in range(mask.shape[1])]


@pytest.fixture(scope="module")
def setup(cuda_device):
    from cgx import exchange

    be = exchange.CudaPackBackend()
    tx = (W + 15) // 16
    bounds = torch.tensor(BOUNDS_ROWS, dtype=torch.int32) * tx
    cams = []
    for k in range(3):
        cpu, gpu = _screen_state(k, cuda_device)
        want = _expected_rows(cpu, bounds)
        ws = len(want)
        wspace = be.workspace(N, ws, cuda_device)
        counts = torch.zeros(ws, dtype=torch.int32, device=cuda_device)
        be.count(gpu[0], gpu[3], bounds.to(cuda_device), H, W, False, counts, wspace)
        cams.append(dict(cpu=cpu, gpu=gpu, want=want, wspace=wspace, counts=counts.cpu()))
    return be, bounds.to(cuda_device), cams


def test_counts_match_oracle_mask(setup):
    _, _, cams = setup
    for c in cams:
        assert c["counts"].tolist() == [len(w) for w in c["want"]]
        assert sum(len(w) for w in c["want"]) > N // 10           # the case actually selects rows


def test_batched_count_equals_per_camera_count(setup, cuda_device):
    """Every camera's counts in two launches, written into one (cameras, ranks) table."""
    be, bounds, cams = setup
    ws = bounds.numel() - 1
    table = torch.full((len(cams), ws), -1, dtype=torch.int32, device=cuda_device)
    spaces = [be.workspace(N, ws, cuda_device) for _ in cams]
    be.count_batched([(c["gpu"][0], c["gpu"][3], bounds, H, W, False, table[k], spaces[k]) for k, c in enumerate(cams)])
    torch.cuda.synchronize()
    for k, c in enumerate(cams):
        assert table[k].cpu().tolist() == c["counts"].tolist()
        used = (N + 255) // 256 * ws * 4                               # bytes of per-tile prefixes (the rest is padding)
        assert torch.equal(spaces[k][:used].cpu(), c["wspace"][:used].cpu())     # what the pack kernel reads


@pytest.mark.parametrize("avoid", [False, True])
def test_mask_equals_reference_kernel(setup, cuda_device, reference_C, avoid):
    """The (P, ws) band mask against the reference's own getTouchedIdsBool (rasterize_points.cu:445-524), bit for
    bit, with and without the one-tile-row widening of `avoid_pixel_all2all`; and the oracle's mask against both."""
    from diff_gaussian_rasterization import _C

    assert reference_C is not None, "oracle/_ref/cityx_ref_C.so is missing: build it with oracle/build_ref.py"
    _, bounds, cams = setup
    args = util.cuda_args()
    args["avoid_pixel_all2all"] = avoid
    ws = bounds.numel() - 1
    for c in cams:
        m2, rad = c["gpu"][0], c["gpu"][3]
        ours = _C.get_local2j_ids_bool(H, W, 0, ws, m2, rad, bounds, args)
        ref = reference_C.get_local2j_ids_bool(H, W, 0, ws, m2, rad, bounds, args)
        assert ours.dtype == torch.bool and ours.shape == ref.shape == (N, ws)
        assert torch.equal(ours, ref)
        assert bool(ref.any()) and not bool(ref.all())
        assert torch.equal(O.local2j_mask(c["cpu"][0], c["cpu"][3], bounds.cpu(), W, H, avoid), ref.cpu())


def _alloc_dsts(want, dev, first_rows):
    """Per destination the eight arrays (with room for first_rows[j] foreign rows in front) and the pointer table."""
    widths = (2, 3, 4, 3, 3, 4, 1, 1)
    arrays, table = [], np.zeros((len(want), 9), dtype=np.uint64)
    for j, rows in enumerate(want):
        n = first_rows[j] + len(rows)
        arrs = [torch.full((n, w), -7.0, device=dev) for w in widths[:6]]
        arrs.append(torch.full((n,), -7, dtype=torch.int32, device=dev))
        arrs.append(torch.full((n,), -7.0, device=dev))
        arrays.append(arrs)
        table[j, :8] = [a.data_ptr() for a in arrs]
        table[j, 8] = first_rows[j]
    return arrays, table


def _check_dsts(arrays, c, first_rows):
    m2, rgb, co, rad, dep, m3, sc, rot = c["cpu"]
    for j, rows in enumerate(c["want"]):
        f = first_rows[j]
        got = [a.cpu() for a in arrays[j]]
        for a, src in zip(got, (m2, rgb, co, m3, sc, rot, rad, dep)):
            assert torch.equal(a[f:], src[rows]), "rows differ from the oracle's selection"
            assert (a[:f] == -7).all(), "rows in front of first_row were overwritten"


def test_direct_store_pack_per_camera_and_batched(setup, cuda_device):
    be, bounds, cams = setup
    first_rows = [5, 0, 11]
    ws = len(first_rows)
    n_send = sum(len(w) for c in cams for w in c["want"])
    # send order: destination major, camera minor
    offs = np.zeros((ws, len(cams)), dtype=np.int64)
    cur = 0
    for j in range(ws):
        for k, c in enumerate(cams):
            offs[j, k] = cur
            cur += len(c["want"][j])
    expect_index = torch.cat([c["want"][j] for j in range(ws) for c in cams]).to(torch.int32)

    # per camera
    idx_a = torch.full((n_send,), -1, dtype=torch.int32, device=cuda_device)
    per_cam = []
    for k, c in enumerate(cams):
        arrays, table = _alloc_dsts(c["want"], cuda_device, first_rows)
        be.pack_p2p(c["gpu"], bounds, H, W, False, table, offs[:, k], idx_a, c["wspace"])
        per_cam.append(arrays)
    torch.cuda.synchronize()
    for arrays, c in zip(per_cam, cams):
        _check_dsts(arrays, c, first_rows)
    assert torch.equal(idx_a.cpu(), expect_index)

    # the whole batch in one launch
    idx_b = torch.full((n_send,), -1, dtype=torch.int32, device=cuda_device)
    batch, all_arrays = [], []
    for k, c in enumerate(cams):
        arrays, table = _alloc_dsts(c["want"], cuda_device, first_rows)
        all_arrays.append(arrays)
        batch.append(dict(params=c["gpu"], bounds=bounds, H=H, W=W, avoid=False, dst_table=table,
                          row_offsets=offs[:, k], workspace=c["wspace"]))
    be.pack_p2p_batched(batch, idx_b)
    torch.cuda.synchronize()
    for arrays, c in zip(all_arrays, cams):
        _check_dsts(arrays, c, first_rows)
    assert torch.equal(idx_b.cpu(), expect_index)


def test_plane_descriptor_record_form(setup, cuda_device):
    """Rows that carry (means2D, rgb, conic_opacity, all_map, radius, depth): 16 floats instead of 21."""
    be, bounds, cams = setup
    first_rows = [3, 0, 2]
    ws = len(first_rows)
    gen = torch.Generator().manual_seed(9)
    batch, all_arrays, maps = [], [], []
    cur, offs_all = 0, []
    for j in range(ws):
        for c in cams:
            offs_all.append(cur)
            cur += len(c["want"][j])
    offs = np.array(offs_all, dtype=np.int64).reshape(ws, len(cams))
    idx = torch.full((cur,), -1, dtype=torch.int32, device=cuda_device)
    for k, c in enumerate(cams):
        am = torch.randn(N, 5, generator=gen)
        maps.append(am)
        arrays, table = [], np.zeros((ws, 10), dtype=np.uint64)
        for j, rows in enumerate(c["want"]):
            n = first_rows[j] + len(rows)
            arrs = [torch.full((n, w), -7.0, device=cuda_device) for w in (2, 3, 4, 5)]
            arrs.append(torch.full((n,), -7, dtype=torch.int32, device=cuda_device))
            arrs.append(torch.full((n,), -7.0, device=cuda_device))
            arrays.append(arrs)
            table[j, [0, 1, 2, 9, 6, 7]] = [a.data_ptr() for a in arrs]
            table[j, 8] = first_rows[j]
        all_arrays.append(arrays)
        m2, rgb, co, rad, dep = c["gpu"][:5]
        batch.append(dict(params=(m2, rgb, co, rad, dep, am.to(cuda_device)), bounds=bounds, H=H, W=W, avoid=False,
                          dst_table=table, row_offsets=offs[:, k], workspace=c["wspace"]))
    be.pack_p2p_batched(batch, idx)
    torch.cuda.synchronize()
    for arrays, c, am in zip(all_arrays, cams, maps):
        m2, rgb, co, rad, dep = c["cpu"][:5]
        for j, rows in enumerate(c["want"]):
            f = first_rows[j]
            for a, src in zip(arrays[j], (m2, rgb, co, am, rad, dep)):
                a = a.cpu()
                assert torch.equal(a[f:], src[rows])
                assert (a[:f] == -7).all()
    assert torch.equal(idx.cpu(), torch.cat([c["want"][j] for j in range(ws) for c in cams]).to(torch.int32))


def test_batched_pack_splits_large_batches(setup, cuda_device):
    """More (camera, rank) pairs than one launch describes: the call must split and still fill every camera."""
    be, bounds, cams = setup
    reps = 18                                   # 18 cameras x 3 ranks = 54 pairs > 48, and > 16 cameras
    first_rows = [0, 0, 0]
    n_send = sum(len(w) for w in cams[0]["want"]) * reps
    idx = torch.full((n_send,), -1, dtype=torch.int32, device=cuda_device)
    c = cams[0]
    per = sum(len(w) for w in c["want"])
    batch, all_arrays = [], []
    for r in range(reps):
        arrays, table = _alloc_dsts(c["want"], cuda_device, first_rows)
        all_arrays.append(arrays)
        offs = np.cumsum([0] + [len(w) for w in c["want"]][:-1]) + r * per
        batch.append(dict(params=c["gpu"], bounds=bounds, H=H, W=W, avoid=False, dst_table=table,
                          row_offsets=offs, workspace=c["wspace"]))
    be.pack_p2p_batched(batch, idx)
    torch.cuda.synchronize()
    for arrays in all_arrays:
        _check_dsts(arrays, c, first_rows)
    one = torch.cat(c["want"]).to(torch.int32)
    assert torch.equal(idx.cpu(), one.repeat(reps))


def test_send_buffer_pack_matches_oracle_mask(setup, cuda_device):
    from cgx.exchange import REC, REC_DIFF

    be, bounds, cams = setup
    c = cams[1]
    n = sum(len(w) for w in c["want"])
    offs = np.cumsum([0] + [len(w) for w in c["want"]][:-1]).tolist()
    send = torch.empty(n, REC_DIFF, device=cuda_device)
    aux = torch.empty(n, REC - REC_DIFF, device=cuda_device)
    idx = torch.empty(n, dtype=torch.int32, device=cuda_device)
    be.pack(c["gpu"], bounds, H, W, False, offs, send, aux, idx, c["wspace"])
    rows = torch.cat(c["want"])
    m2, rgb, co, rad, dep, m3, sc, rot = c["cpu"]
    assert torch.equal(send.cpu(), torch.cat([m2, rgb, co, m3, sc, rot], 1)[rows])
    assert torch.equal(aux.cpu(), torch.stack([rad.float(), dep], 1)[rows])
    assert torch.equal(idx.cpu(), rows.to(torch.int32))


@pytest.mark.parametrize("ncols", [9, 14, 19])
def test_gradient_rows_round_trip(setup, cuda_device, ncols):
    """Receiver side: cotangents of one camera's received rows -> per-source segments; owner side: segments
    scatter-added through the send index.  A row sent to two ranks gets both contributions.  Row widths: 19 = all
    differentiable columns, 9 = screen-space only, 14 = screen-space + plane descriptors (in the means3D slot)."""
    be, bounds, cams = setup
    c = cams[2]
    want = c["want"]
    gen = torch.Generator().manual_seed(5)
    widths = {19: (2, 3, 4, 3, 3, 4), 9: (2, 3, 4), 14: (2, 3, 4, 5)}[ncols]
    pad = [None] * (6 - len(widths))
    staging = torch.zeros(sum(len(w) for w in want), ncols, device=cuda_device)
    expect = [torch.zeros(N, w, dtype=torch.float64) for w in widths]
    start = 0
    for rows in want:                      # every destination returns one segment of gradient rows
        n = len(rows)
        cot = [torch.randn(n, w, generator=gen) for w in widths]
        seg_ptr = staging.data_ptr() + start * ncols * 4
        be.pack_grad_rows_to([seg_ptr], [n], ncols, [t.to(cuda_device) for t in cot] + pad)
        for e, t in zip(expect, cot):
            e.index_add_(0, rows, t.double())
        start += n
    index = torch.cat(want).to(torch.int32).to(cuda_device)
    grads = [torch.zeros(N, w, device=cuda_device) for w in widths]
    ranges, s = [], 0
    for rows in want:
        ranges.append((s, s + len(rows)))
        s += len(rows)
    be.unpack_grad_add_cols(staging, index, ranges, ncols, grads + pad)
    for g, e in zip(grads, expect):
        assert torch.allclose(g.cpu().double(), e, atol=1e-5, rtol=1e-6)


@pytest.mark.parametrize("first", [0, 1, 2, 3])
def test_gradient_rows_to_several_owners_in_any_starting_order(cuda_device, first):
    """One launch of cgx_pack_grad_rows_to with four segments (one empty): whichever segment the grid starts with,
    every segment receives exactly its rows."""
    from cgx import exchange

    be = exchange.default_backend()
    gen = torch.Generator().manual_seed(11)
    counts = [700, 0, 1300, 257]
    n = sum(counts)
    cot = [torch.randn(n, w, generator=gen).to(cuda_device) for w in (2, 3, 4, 5)]
    segs = [torch.full((max(c, 1), 14), float("nan"), device=cuda_device) for c in counts]
    be.pack_grad_rows_to([s.data_ptr() for s in segs], counts, 14, cot + [None, None], first_segment=first)
    torch.cuda.synchronize()
    want = torch.cat(cot, 1)
    start = 0
    for s, c in zip(segs, counts):
        if c:
            assert torch.equal(s[:c], want[start:start + c])
        start += c
