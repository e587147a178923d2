"""Per-batch Gaussian all-to-all: every rank sends, for every camera, the screen-space records of its local
Gaussians to the ranks whose tile-row band they touch.

Drop-in for ``all_to_all_communication_final`` of the reference (gaussian_renderer/__init__.py:600-786) with
the same inputs, the same outputs and the same row order (per camera: source rank ascending, within a source
ascending local index; a Gaussian straddling a cut goes to both neighbours), but a different mechanism:

  reference                                             here
  ---------                                             ----
  (P, ws) bool mask + ws x nonzero() per camera         one counting kernel per camera, ONE host read of all
  (ws x bsz host synchronisations)                      counts of the batch
  index-gather + cat per (destination, camera)          one packing kernel per camera writes 21-float rows
  in Python, two record tensors (19 + 2 floats)         [19 differentiable | radius | depth] straight into the
                                                        per-destination segments of one send buffer
  list all_to_all x2 (functional + plain)               one ``all_to_all_single`` with split sizes (NCCL over
                                                        NVLink; works on gloo as well)
  backward: autograd through functional all_to_all,     one reverse ``all_to_all_single`` of 19-float gradient
  index_put / cat backward kernels                      rows + one scatter-add kernel through the saved
                                                        source-row index

The packing backend is injected (`backend=`): the product backend drives the CUDA kernels of the C ABI
(cgx_local2j_count / cgx_local2j_pack / cgx_unpack_grad_add) and refuses CPU tensors; the CPU tests inject
their own checker backend to exercise this module's host logic on gloo.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

REC = 21          # floats per travelling row
REC_DIFF = 19     # of which differentiable: means2D 2 | rgb 3 | conic_opacity 4 | means3D 3 | scales 3 | rotation 4
SPLITS = [2, 3, 4, 3, 3, 4]


class CudaPackBackend:
    """Counting / packing / gradient scatter on the GPU through the C ABI."""

    def __init__(self):
        from diff_gaussian_rasterization import _lib

        self._lib = _lib
        self.l = _lib.lib()

    @staticmethod
    def _p(t):
        return None if t is None else C.c_void_p(t.data_ptr())

    @staticmethod
    def _st():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _require_cuda(self, t):
        if not t.is_cuda:
            raise RuntimeError("cgx.exchange: the packing backend needs CUDA tensors (no CPU path)")

    def workspace(self, P, ws, device):
        return torch.empty(max(1, self.l.cgx_local2j_workspace_bytes(P, ws)), dtype=torch.uint8, device=device)

    def count(self, means2D, radii, tile_bounds, H, W, avoid, counts_out, workspace):
        self._require_cuda(means2D)
        P, ws = means2D.shape[0], tile_bounds.numel() - 1
        self._lib.check(self.l.cgx_local2j_count(P, H, W, ws, self._p(means2D), self._p(radii), self._p(tile_bounds),
                                                 int(avoid), self._p(counts_out), self._p(workspace),
                                                 workspace.numel(), self._st()), "cgx_local2j_count")

    def pack(self, params, tile_bounds, H, W, avoid, row_offsets, send, send_aux, send_index, workspace):
        means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation = [t.contiguous() for t in params]
        P, ws = means2D.shape[0], tile_bounds.numel() - 1
        offs = (C.c_int64 * ws)(*[int(o) for o in row_offsets])
        self._lib.check(self.l.cgx_local2j_pack(
            P, H, W, ws, self._p(means2D), self._p(rgb), self._p(conic_opacity), self._p(means3D), self._p(scales),
            self._p(rotation), self._p(radii), self._p(depths), self._p(tile_bounds), int(avoid), offs, self._p(send),
            self._p(send_aux), self._p(send_index), self._p(workspace), workspace.numel(), self._st()),
            "cgx_local2j_pack")

    def unpack_grad_add(self, grad_rows, send_index, ranges, grads):
        """ranges: list of (start, stop) row ranges of grad_rows that belong to one camera."""
        ranges = [(a, b) for a, b in ranges if b > a]
        if not ranges:
            return
        n = len(ranges)
        starts = (C.c_int64 * n)(*[a for a, _ in ranges])
        stops = (C.c_int64 * n)(*[b for _, b in ranges])
        d_m2, d_rgb, d_co, d_m3, d_sc, d_rot = grads
        self._lib.check(self.l.cgx_unpack_grad_add(n, starts, stops, self._p(grad_rows), self._p(send_index),
                                                   self._p(d_m2), self._p(d_rgb), self._p(d_co), self._p(d_m3),
                                                   self._p(d_sc), self._p(d_rot), self._st()), "cgx_unpack_grad_add")


_default_backend = None


def default_backend():
    global _default_backend
    if _default_backend is None:
        _default_backend = CudaPackBackend()
    return _default_backend


def _world(group):
    return dist.get_world_size(group), dist.get_rank(group)


def _gather_sizes(local_sizes, group, device):
    """local_sizes: (ws, bsz) int32 rows = destination rank -> (ws, ws, bsz) nested list [src][dst][cam]."""
    ws = dist.get_world_size(group)
    backend = dist.get_backend(group)
    t = local_sizes.to(device if backend == "nccl" else "cpu").contiguous().view(-1)
    out = torch.empty(ws * t.numel(), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t, group=group)
    return out.view(ws, ws, -1).cpu()


class _Exchange(torch.autograd.Function):
    """send rows (n_send, 19) -> received rows (n_recv, 19); backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, send_diff, send_splits, recv_splits, group):
        ctx.group, ctx.send_splits, ctx.recv_splits = group, send_splits, recv_splits
        recv = send_diff.new_empty((sum(recv_splits), send_diff.shape[1]))
        dist.all_to_all_single(recv, send_diff.contiguous(), output_split_sizes=recv_splits,
                               input_split_sizes=send_splits, group=group)
        return recv

    @staticmethod
    def backward(ctx, grad_recv):
        grad_send = grad_recv.new_empty((sum(ctx.send_splits), grad_recv.shape[1]))
        dist.all_to_all_single(grad_send, grad_recv.contiguous(), output_split_sizes=ctx.send_splits,
                               input_split_sizes=ctx.recv_splits, group=ctx.group)
        return grad_send, None, None, None


class _PackRows(torch.autograd.Function):
    """Differentiable view of the packing kernel: flat per-camera inputs -> (n_send, 19) rows.

    forward receives the already packed buffer (packing is fused with selection in one kernel); backward
    scatter-adds the row gradients back onto the per-camera source tensors through the saved source index."""

    @staticmethod
    def forward(ctx, packed_diff, cam_of_row_ranges, send_index, backend, *flat_inputs):
        ctx.backend, ctx.ranges = backend, cam_of_row_ranges
        ctx.shapes = [t.shape for t in flat_inputs]
        ctx.save_for_backward(send_index)
        return packed_diff.view_as(packed_diff)

    @staticmethod
    def backward(ctx, grad_rows):
        (send_index,) = ctx.saved_tensors
        grad_rows = grad_rows.contiguous()
        grads = [torch.zeros(s, dtype=grad_rows.dtype, device=grad_rows.device) for s in ctx.shapes]
        # rows of camera k occupy, per destination, the range ctx.ranges[k][..] = (start, stop) of the send buffer
        for k, per_dst in enumerate(ctx.ranges):
            ctx.backend.unpack_grad_add(grad_rows, send_index, per_dst, grads[6 * k: 6 * k + 6])
        return (None, None, None, None) + tuple(grads)


def all_to_all_communication_final(batched_rasterizers, batched_screenspace_params, batched_cuda_args,
                                   batched_strategies, group=None, backend=None):
    """See module docstring.  ``batched_screenspace_params[k]`` =
    (means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation) of camera k on this rank.

    Returns the reference's tuple: per-camera lists of means2D, rgb, conic_opacity, radii (int32), depths, means3D,
    scales, rotations (redistributed), then the size table [src][dst][cam] and, per destination and camera, the
    number of rows sent (the reference returns index tensors there; here the source indices stay on the device in
    one packed tensor, which is returned as the last element)."""
    backend = backend or default_backend()
    ws, me = _world(group)
    bsz = len(batched_rasterizers)
    dev = batched_screenspace_params[0][0].device

    # ---- 1. counts: one kernel per camera, results land in one (ws, bsz) table, one host read
    counts_dev = torch.zeros(bsz, ws, dtype=torch.int32, device=dev)
    scratch, bounds = [], []
    for k in range(bsz):
        strat = batched_strategies[k]
        rs = batched_rasterizers[k].raster_settings
        means2D, radii = batched_screenspace_params[k][0], batched_screenspace_params[k][3]
        tb = strat.tile_bounds(dev)
        wsk = len(strat.gpu_ids)
        wspace = backend.workspace(means2D.shape[0], wsk, dev)
        g0 = strat.gpu_ids[0]
        contiguous_ranks = list(strat.gpu_ids) == list(range(g0, g0 + wsk))
        c = counts_dev[k, g0:g0 + wsk] if contiguous_ranks else torch.zeros(wsk, dtype=torch.int32, device=dev)
        backend.count(means2D.detach().contiguous(), radii.contiguous(), tb, rs.image_height, rs.image_width,
                      batched_cuda_args[k]["avoid_pixel_all2all"], c, wspace)
        if not contiguous_ranks:
            counts_dev[k, torch.as_tensor(strat.gpu_ids, device=dev, dtype=torch.long)] = c
        scratch.append(wspace)
        bounds.append(tb)
    local_sizes = counts_dev.t().contiguous()                      # (dst, cam)
    sizes = _gather_sizes(local_sizes, group, dev)                 # (src, dst, cam) on the host
    sizes_list = sizes.tolist()
    my = sizes[me]                                                 # (dst, cam)

    # ---- 2. layout of the send buffer: destination major, camera minor
    send_splits = [int(my[j].sum()) for j in range(ws)]
    recv_splits = [int(sizes[i, me].sum()) for i in range(ws)]
    n_send, n_recv = sum(send_splits), sum(recv_splits)
    dst_base = [0] * ws
    for j in range(1, ws):
        dst_base[j] = dst_base[j - 1] + send_splits[j - 1]
    send = torch.empty(n_send, REC_DIFF, dtype=torch.float32, device=dev)
    send_aux = torch.empty(n_send, REC - REC_DIFF, dtype=torch.float32, device=dev)
    send_index = torch.empty(n_send, dtype=torch.int32, device=dev)
    ranges = []
    cam_off = [0] * ws                                             # rows of earlier cameras per destination
    for k in range(bsz):
        strat = batched_strategies[k]
        offs = [dst_base[j] + cam_off[j] for j in strat.gpu_ids]
        params = tuple(t.detach() for t in batched_screenspace_params[k])
        rs = batched_rasterizers[k].raster_settings
        backend.pack(params, bounds[k], rs.image_height, rs.image_width,
                     batched_cuda_args[k]["avoid_pixel_all2all"], offs, send, send_aux, send_index, scratch[k])
        per_dst = []
        for j in strat.gpu_ids:
            n = int(my[j, k])
            per_dst.append((dst_base[j] + cam_off[j], dst_base[j] + cam_off[j] + n))
            cam_off[j] += n
        ranges.append(per_dst)

    # ---- 3. exchange: 19 differentiable columns through autograd, the 2 auxiliary columns plainly
    flat = []
    for k in range(bsz):
        m2, rgb, co, radii, depths, m3, sc, rot = batched_screenspace_params[k]
        flat += [m2, rgb, co, m3, sc, rot]
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in flat)
    send_diff = send
    if needs_grad:
        send_diff = _PackRows.apply(send_diff, ranges, send_index, backend, *flat)
        recv_diff = _Exchange.apply(send_diff, send_splits, recv_splits, group)
    else:
        recv_diff = send.new_empty((n_recv, REC_DIFF))
        dist.all_to_all_single(recv_diff, send_diff.contiguous(), output_split_sizes=recv_splits,
                               input_split_sizes=send_splits, group=group)
    recv_aux = send.new_empty((n_recv, REC - REC_DIFF))
    dist.all_to_all_single(recv_aux, send_aux, output_split_sizes=recv_splits,
                           input_split_sizes=send_splits, group=group)

    # ---- 4. per camera: concatenate the blocks of all sources (source rank ascending)
    src_base = [0] * ws
    for i in range(1, ws):
        src_base[i] = src_base[i - 1] + recv_splits[i - 1]
    out = [[] for _ in range(8)]
    cam_off = [0] * ws
    for k in range(bsz):
        idx = []
        for i in range(ws):
            n = sizes_list[i][me][k]
            a = src_base[i] + cam_off[i]
            idx.append((a, a + n))
            cam_off[i] += n
        rows = torch.cat([recv_diff[a:b] for a, b in idx], dim=0) if ws > 1 else recv_diff[idx[0][0]:idx[0][1]]
        aux = torch.cat([recv_aux[a:b] for a, b in idx], dim=0) if ws > 1 else recv_aux[idx[0][0]:idx[0][1]]
        m2, rgb, co, m3, sc, rot = torch.split(rows, SPLITS, dim=1)
        out[0].append(m2.contiguous())
        out[1].append(rgb.contiguous())
        out[2].append(co.contiguous())
        out[3].append(aux[:, 0].int())
        out[4].append(aux[:, 1].contiguous())
        out[5].append(m3.contiguous())
        out[6].append(sc.contiguous())
        out[7].append(rot.contiguous())
    sent_counts = [[sizes_list[me][j][k] for k in range(bsz)] for j in range(ws)]
    stats = {"rows_sent": n_send, "rows_received": n_recv, "bytes_sent_fwd": n_send * REC * 4,
             "bytes_sent_bwd": n_send * REC_DIFF * 4}
    return (*out, sizes_list, sent_counts, send_index, stats)
