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
  split + cat per camera on the receiver               one unpack kernel per camera writes the contiguous
                                                        per-camera tensors
  backward: autograd through functional all_to_all,     ONE autograd node: gradient rows packed by one kernel
  split / cat / index backward kernels                  per camera, one reverse ``all_to_all_single`` of
                                                        19-float rows, one scatter-add kernel per camera
                                                        through the saved source-row index

Two transports share the planning code.  ``collective`` (any backend): pack kernel -> ``all_to_all_single``
-> unpack kernel, as tabulated above.  ``p2p`` (NCCL groups inside one NVLink/NVSwitch domain, the default there):
the ranks' receive arenas are symmetric memory mapped into every peer, and ONE kernel per camera does selection,
packing and transport by storing each selected row straight into the final per-camera tensors of the rank that
renders it (`cgx_local2j_pack_p2p`); the backward stores gradient rows straight into the source rank's staging
buffer (`cgx_pack_grad_rows_to`).  Stream-ordered device barriers (symmetric-memory signal pads) order writers
and readers; no send buffer, no collective, no unpack.  Tensors returned in this mode are views of one of two
receive arenas that alternate exchanges use: they stay valid until the exchange after the next one of the group.

The packing backend is injected (`backend=`): the product backend drives the CUDA kernels of the C ABI
(cgx_local2j_count / cgx_local2j_pack / cgx_unpack_grad_add) and refuses CPU tensors; the CPU tests inject
their own checker backend to exercise this module's host logic on gloo.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
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
        from diff_gaussian_rasterization._lib import current_stream_ptr

        return current_stream_ptr()

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

    def count_batched(self, cameras):
        """cameras: list of (means2D, radii, tile_bounds, H, W, avoid, counts_out, workspace): two launches for all."""
        table = np.zeros((len(cameras), 11), dtype=np.uint64)          # rows = struct cgx_count_camera
        for k, (means2D, radii, tb, H, W, avoid, counts_out, workspace) in enumerate(cameras):
            self._require_cuda(means2D)
            table[k] = (means2D.shape[0], H, W, tb.numel() - 1, means2D.data_ptr(), radii.data_ptr(), tb.data_ptr(),
                        int(bool(avoid)), counts_out.data_ptr(), workspace.data_ptr(), workspace.numel())
        self._lib.check(self.l.cgx_local2j_count_batched(len(cameras), C.c_void_p(table.ctypes.data), self._st()),
                        "cgx_local2j_count_batched")

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


    def unpack_rows(self, segments, recv, recv_aux, outs):
        n = len(segments)
        if n == 0:
            return
        starts = (C.c_int64 * n)(*[a for a, _ in segments])
        counts = (C.c_int64 * n)(*[c for _, c in segments])
        m2, rgb, co, rad, dep, m3, sc, rot = outs
        self._lib.check(self.l.cgx_unpack_rows(n, starts, counts, self._p(recv), self._p(recv_aux), self._p(m2),
                                               self._p(rgb), self._p(co), self._p(m3), self._p(sc), self._p(rot),
                                               self._p(rad), self._p(dep), self._st()), "cgx_unpack_rows")

    def pack_grad_rows(self, segments, grads, rows):
        n = len(segments)
        if n == 0:
            return
        starts = (C.c_int64 * n)(*[a for a, _ in segments])
        counts = (C.c_int64 * n)(*[c for _, c in segments])
        g = [None if t is None else t.contiguous() for t in grads]
        self._lib.check(self.l.cgx_pack_grad_rows(n, starts, counts, *[self._p(t) for t in g], self._p(rows),
                                                  self._st()), "cgx_pack_grad_rows")


    def pack_p2p(self, params, tile_bounds, H, W, avoid, dst_table, row_offsets, send_index, workspace):
        """dst_table: (ws, 9) uint64 rows = the eight destination tensors' device addresses (means2D, rgb,
        conic_opacity, means3D, scales, rotations, radii, depths) and the first row this rank writes there, i.e.
        an array of `struct cgx_peer_camera_dst`."""
        means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation = [t.contiguous() for t in params]
        P, ws = means2D.shape[0], tile_bounds.numel() - 1
        dst_table = _dst_rows(dst_table, ws)
        offs = (C.c_int64 * ws)(*[int(o) for o in row_offsets])
        self._lib.check(self.l.cgx_local2j_pack_p2p(
            P, H, W, ws, self._p(means2D), self._p(rgb), self._p(conic_opacity), self._p(means3D), self._p(scales),
            self._p(rotation), self._p(radii), self._p(depths), self._p(tile_bounds), int(avoid),
            C.c_void_p(dst_table.ctypes.data), offs, self._p(send_index), self._p(workspace), workspace.numel(),
            self._st()), "cgx_local2j_pack_p2p")

    def pack_p2p_batched(self, cameras, send_index):
        """One launch for the whole batch.  cameras: list of dicts with keys params (the eight per-camera tensors, or
        six in the plane-descriptor form: means2D, rgb, conic_opacity, radii, depths, all_map), bounds, H, W, avoid,
        dst_table ((ws_k, 9 or 10) uint64, see pack_p2p), row_offsets ((ws_k,) int64), workspace."""
        n = len(cameras)
        table = np.zeros((n, 19), dtype=np.uint64)          # rows = struct cgx_exchange_camera
        keep = []
        for k, c in enumerate(cameras):
            params = [t.contiguous() for t in c["params"]]
            if len(params) == 6:
                means2D, rgb, conic_opacity, radii, depths, all_map = params
                m3 = sc = rot = am = 0
                am = all_map.data_ptr()
            else:
                means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation = params
                m3, sc, rot, am = means3D.data_ptr(), scales.data_ptr(), rotation.data_ptr(), 0
            ws = c["bounds"].numel() - 1
            dst = _dst_rows(c["dst_table"], ws)
            offs = np.ascontiguousarray(c["row_offsets"], dtype=np.int64)
            assert offs.shape == (ws,)
            keep.append((params, dst, offs))
            table[k] = (means2D.shape[0], c["H"], c["W"], ws, means2D.data_ptr(), rgb.data_ptr(),
                        conic_opacity.data_ptr(), m3, sc, rot, radii.data_ptr(), depths.data_ptr(),
                        c["bounds"].data_ptr(), int(bool(c["avoid"])), dst.ctypes.data, offs.ctypes.data,
                        c["workspace"].data_ptr(), c["workspace"].numel(), am)
        from diff_gaussian_rasterization import _C          # per-stage events when a profile is being collected

        _C._call("cgx_local2j_pack_p2p_batched", self.l.cgx_local2j_pack_p2p_batched, n,
                 C.c_void_p(table.ctypes.data), self._p(send_index), self._st())
        del keep

    def prepare_pack_p2p(self, cameras, order):
        """Everything of `pack_p2p_batched` that does not depend on the size table: `cameras` as there, without
        dst_table / row_offsets; `order` = the order in which the launch works through the cameras.  Returns the
        object `pack_p2p_prepared` takes."""
        n = len(cameras)
        table = np.zeros((n, 19), dtype=np.uint64)          # rows = struct cgx_exchange_camera
        keep, n_dst = [], []
        for row, k in enumerate(order):
            c = cameras[k]
            params = [t.contiguous() for t in c["params"]]
            if len(params) == 6:
                means2D, rgb, conic_opacity, radii, depths, all_map = params
                m3 = sc = rot = 0
                am = all_map.data_ptr()
            else:
                means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation = params
                m3, sc, rot, am = means3D.data_ptr(), scales.data_ptr(), rotation.data_ptr(), 0
            ws = c["bounds"].numel() - 1
            keep.append(params)
            n_dst.append(ws)
            table[row] = (means2D.shape[0], c["H"], c["W"], ws, means2D.data_ptr(), rgb.data_ptr(),
                          conic_opacity.data_ptr(), m3, sc, rot, radii.data_ptr(), depths.data_ptr(),
                          c["bounds"].data_ptr(), int(bool(c["avoid"])), 0, 0,
                          c["workspace"].data_ptr(), c["workspace"].numel(), am)
        entry0 = np.concatenate([[0], np.cumsum(n_dst)]).astype(np.int64)
        return dict(table=table, keep=keep, entry0=entry0, n=n)

    def pack_p2p_prepared(self, prep, dst_rows, row_offsets, send_index):
        """The launch of `pack_p2p_batched` from a prepared table: dst_rows (entries, 10) uint64 and row_offsets
        (entries,) int64 hold the cameras' destination rows one camera after the other, in the prepared order."""
        table, entry0 = prep["table"], prep["entry0"]
        dst_rows = np.ascontiguousarray(dst_rows, dtype=np.uint64)
        row_offsets = np.ascontiguousarray(row_offsets, dtype=np.int64)
        assert dst_rows.shape == (int(entry0[-1]), 10) and row_offsets.shape == (int(entry0[-1]),)
        table[:, 14] = (dst_rows.ctypes.data + entry0[:-1] * 80).astype(np.uint64)
        table[:, 15] = (row_offsets.ctypes.data + entry0[:-1] * 8).astype(np.uint64)
        from diff_gaussian_rasterization import _C

        _C._call("cgx_local2j_pack_p2p_batched", self.l.cgx_local2j_pack_p2p_batched, prep["n"],
                 C.c_void_p(table.ctypes.data), self._p(send_index), self._st())

    def pack_grad_rows_to(self, seg_ptrs, seg_counts, ncols, grads, first_segment=0):
        n = len(seg_ptrs)
        if n == 0 or sum(seg_counts) == 0:
            return
        ptrs = (C.c_void_p * n)(*seg_ptrs)
        counts = (C.c_int64 * n)(*seg_counts)
        g = [None if t is None else t.contiguous() for t in grads]
        from diff_gaussian_rasterization import _C

        _C._call("cgx_pack_grad_rows_to", self.l.cgx_pack_grad_rows_to, n, ptrs, counts, ncols,
                 int(first_segment) % n, *[self._p(t) for t in g], self._st())

    def unpack_grad_add_cols(self, grad_rows, send_index, ranges, ncols, grads):
        ranges = [(a, b) for a, b in ranges if b > a]
        if not ranges:
            return
        n = len(ranges)
        starts = (C.c_int64 * n)(*[a for a, _ in ranges])
        stops = (C.c_int64 * n)(*[b for _, b in ranges])
        d_m2, d_rgb, d_co, d_m3, d_sc, d_rot = grads
        self._lib.check(self.l.cgx_unpack_grad_add_cols(n, starts, stops, ncols, self._p(grad_rows),
                                                        self._p(send_index), self._p(d_m2), self._p(d_rgb),
                                                        self._p(d_co), self._p(d_m3), self._p(d_sc), self._p(d_rot),
                                                        self._st()), "cgx_unpack_grad_add_cols")


def _dst_rows(dst_table, ws):
    """(ws, 10) uint64 rows = struct cgx_peer_camera_dst; a 9-column table (no plane descriptors) is padded."""
    t = np.asarray(dst_table, dtype=np.uint64)
    if t.shape == (ws, 9):
        t = np.concatenate([t, np.zeros((ws, 1), dtype=np.uint64)], axis=1)
    assert t.shape == (ws, 10)
    return np.ascontiguousarray(t)


_default_backend = None


def default_backend():
    global _default_backend
    if _default_backend is None:
        _default_backend = CudaPackBackend()
    return _default_backend


_world_cache = {}


def _world(group):
    key = id(group)
    if key not in _world_cache:
        _world_cache[key] = (dist.get_world_size(group), dist.get_rank(group))
    return _world_cache[key]


_pinned = {}


def _gather_table(table, n_counts, piggyback, group, ws, overlap=None):
    """All-gather every rank's `table` (int32: n_counts row counts, then len(piggyback) float32 bit patterns) and
    read it on the host: the one host synchronisation of the exchange.  Returns (int64 array (ws, n_counts),
    nested list (ws, len(piggyback)) of floats).  `overlap`: called after the read-back has been queued and before
    the host waits for it, for launches that do not depend on the table (they run while the host plans)."""
    L = table.numel() - n_counts
    if L:
        if table.is_cuda:
            stage = _pinned.get(L)
            if stage is None:
                stage = _pinned[L] = torch.empty(L, dtype=torch.float32).pin_memory()
            stage.numpy()[:] = np.asarray(piggyback, dtype=np.float32)
            # the staging buffer is free again after the host read below, i.e. before the next call fills it
            table[n_counts:].view(torch.float32).copy_(stage, non_blocking=True)
        else:
            table[n_counts:].view(torch.float32).copy_(torch.tensor(list(piggyback), dtype=torch.float32))
    out = torch.empty(ws * table.numel(), dtype=torch.int32, device=table.device)
    dist.all_gather_into_tensor(out, table, group=group)
    if out.is_cuda:
        stage = _pinned.get(("table", out.numel()))
        if stage is None:
            stage = _pinned[("table", out.numel())] = torch.empty(out.numel(), dtype=torch.int32).pin_memory()
        from diff_gaussian_rasterization import _lib

        # carried by a kernel: a copy-engine transfer would queue behind bulk read-backs of other streams
        _lib.check(_lib.lib().cgx_post_words(C.c_void_p(out.data_ptr()), C.c_void_p(stage.data_ptr()), out.numel(),
                                             _lib.current_stream_ptr()), "cgx_post_words")
        status = _queue_status_read()
        ev = torch.cuda.Event()
        ev.record()
        if overlap is not None:
            overlap()
        ev.synchronize()
        _raise_on_device_status(status)
        host = stage.numpy().reshape(ws, -1).copy()
    else:
        if overlap is not None:
            overlap()
        host = out.numpy().reshape(ws, -1)
    extra = host[:, n_counts:].copy().view(np.float32).tolist() if L else [[] for _ in range(ws)]
    return host[:, :n_counts].astype(np.int64), extra


def _queue_status_read():
    """Queue a copy of the library's device status words (set when a bounded device-side wait gave up) into pinned
    memory, in front of a host synchronisation the caller performs anyway."""
    from diff_gaussian_rasterization import _lib

    stage = _pinned.get("status")
    if stage is None:
        stage = _pinned["status"] = torch.zeros(4, dtype=torch.int32).pin_memory()
    _lib.check(_lib.lib().cgx_device_status_async(C.c_void_p(stage.data_ptr()), _lib.current_stream_ptr()),
               "cgx_device_status_async")
    return stage


def _raise_on_device_status(stage):
    """After the synchronisation: a wait that ran out earlier on this stream (a peer that never signalled, a bulk
    copy that never completed) means rows may not have landed, so the step must not go on silently."""
    if stage[0].item() or stage[1].item() or stage[2].item():
        from diff_gaussian_rasterization import _lib

        code = C.c_int(0)
        _lib.lib().cgx_device_status(C.byref(code), _lib.current_stream_ptr())      # reads and clears
        where = "the blending kernels" if stage[0].item() else \
            ("the peer barrier of the Gaussian exchange" if stage[1].item() else "the sort's look-back")
        raise _lib.CgxError(_lib.CGX_ETIMEDOUT, f"a bounded device-side wait in {where}")


def _dense_cotangents(g8, n, dev):
    """The six differentiable outputs' cotangents of one camera; the first three (means2D, rgb, conic_opacity) are
    always read by the packing kernels, so an output nothing consumed gets zeros; the 3-D ones may stay None."""
    widths = (2, 3, 4)
    first = [g if g is not None else torch.zeros(n, w, dtype=torch.float32, device=dev)
             for g, w in zip(g8[:3], widths)]
    return (*first, g8[5], g8[6], g8[7])


class _GaussianExchange(torch.autograd.Function):
    """The whole exchange as one autograd node.

    inputs : plan, then 6 differentiable tensors per camera (means2D, rgb, conic_opacity, means3D, scales, rotation)
    outputs: 8 tensors per camera (means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation)
    """

    @staticmethod
    def forward(ctx, plan, *flat):
        be, group = plan["backend"], plan["group"]
        send, send_aux = plan["send"], plan["send_aux"]
        n_recv = sum(plan["recv_splits"])
        recv = send.new_empty((n_recv, REC_DIFF))
        recv_aux = send.new_empty((n_recv, REC - REC_DIFF))
        dist.all_to_all_single(recv, send, output_split_sizes=plan["recv_splits"],
                               input_split_sizes=plan["send_splits"], group=group)
        dist.all_to_all_single(recv_aux, send_aux, output_split_sizes=plan["recv_splits"],
                               input_split_sizes=plan["send_splits"], group=group)
        outs, nondiff = [], []
        for segs in plan["recv_segments"]:
            n = sum(c for _, c in segs)
            f = dict(dtype=torch.float32, device=send.device)
            o = (recv.new_empty((n, 2)), recv.new_empty((n, 3)), recv.new_empty((n, 4)),
                 torch.empty(n, dtype=torch.int32, device=send.device), torch.empty(n, **f),
                 recv.new_empty((n, 3)), recv.new_empty((n, 3)), recv.new_empty((n, 4)))
            be.unpack_rows(segs, recv, recv_aux, o)
            outs += list(o)
            nondiff += [o[3], o[4]]
        ctx.plan = plan
        ctx.shapes = [t.shape for t in flat]
        ctx.mark_non_differentiable(*nondiff)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *gouts):
        plan = ctx.plan
        be, group = plan["backend"], plan["group"]
        dev = plan["send"].device
        n_recv, n_send = sum(plan["recv_splits"]), sum(plan["send_splits"])
        grad_recv = torch.empty((n_recv, REC_DIFF), dtype=torch.float32, device=dev)
        for k, segs in enumerate(plan["recv_segments"]):
            g8 = gouts[8 * k: 8 * k + 8]
            n = sum(c for _, c in segs)
            if n:
                be.pack_grad_rows(segs, _dense_cotangents(g8, n, dev), grad_recv)
        grad_send = torch.empty((n_send, REC_DIFF), dtype=torch.float32, device=dev)
        dist.all_to_all_single(grad_send, grad_recv, output_split_sizes=plan["send_splits"],
                               input_split_sizes=plan["recv_splits"], group=group)
        grads = []
        for k, per_dst in enumerate(plan["send_ranges"]):
            need = ctx.needs_input_grad[1 + 6 * k: 1 + 6 * k + 6]
            g6 = [torch.zeros(s, dtype=torch.float32, device=dev) if nd else None
                  for s, nd in zip(ctx.shapes[6 * k: 6 * k + 6], need)]
            if g6[0] is None or g6[2] is None:       # the scatter kernel always writes means2D and conic_opacity
                g6[0] = g6[0] if g6[0] is not None else torch.zeros(ctx.shapes[6 * k], dtype=torch.float32, device=dev)
                g6[2] = g6[2] if g6[2] is not None else torch.zeros(ctx.shapes[6 * k + 2], dtype=torch.float32, device=dev)
            be.unpack_grad_add(grad_send, plan["send_index"], per_dst, g6)
            grads += [g if nd else None for g, nd in zip(g6, need)]
        return (None,) + tuple(grads)



def _align_up(v, a=256):
    return (v + a - 1) // a * a


# per-camera tensors of a receive region: (name, bytes per row), in arena order
_CAM_FIELDS = (("means2D", 8), ("rgb", 12), ("conic_opacity", 16), ("means3D", 12), ("scales", 12), ("rotations", 16),
               ("radii", 4), ("depths", 4))
_CAM_FIELDS_PLANES = (("means2D", 8), ("rgb", 12), ("conic_opacity", 16), ("all_map", 20), ("radii", 4), ("depths", 4))


def _camera_layouts(n_rows, fields=_CAM_FIELDS):
    """For an integer array of row counts (any shape): byte offsets of the per-camera tensors inside an arena
    region (shape + (len(fields),)) and the region sizes (same shape).  Every tensor starts on a 256-byte boundary."""
    widths = np.array([w for _, w in fields], dtype=np.int64)
    nbytes = (np.asarray(n_rows, dtype=np.int64)[..., None] * widths + 255) // 256 * 256
    ends = np.cumsum(nbytes, axis=-1)
    return ends - nbytes, ends[..., -1]


def _camera_layout(n, fields=_CAM_FIELDS):
    offs, size = _camera_layouts(n, fields)
    return [int(o) for o in offs], int(size)


def p2p_layout(S, me, fields=_CAM_FIELDS):
    """Where everything goes in the peer-to-peer exchange, from the gathered size table S[src, dst, cam] (pure
    integer arithmetic, the same on every rank except for the rows that depend on `me`):

    n_recv[dst, cam]       rows rank dst receives for camera cam (all sources)
    cam_base[dst, cam]     byte offset of camera cam's region in rank dst's receive arena
    field_off[dst, cam, f] byte offset of tensor f inside that region (256-byte aligned)
    recv_bytes             arena size that holds every rank's regions
    first_row[dst, cam]    first row rank `me` writes in (dst, cam)'s tensors: behind the rows of lower source ranks
    grad_row[src, cam]     row, in rank src's gradient staging buffer (= its send order: destination major, camera
                           minor), of the segment whose gradients rank `me` returns to src for camera cam
    grad_rows_max          rows of the largest staging buffer
    """
    S = np.asarray(S, dtype=np.int64)
    ws, _, bsz = S.shape
    n_recv = S.sum(0)
    field_off, cam_size = _camera_layouts(n_recv, fields)
    cam_end = np.cumsum(cam_size, axis=1)
    per_src = S.reshape(ws, -1)
    grad_row = (np.cumsum(per_src, axis=1) - per_src).reshape(ws, ws, bsz)[:, me, :]
    return dict(n_recv=n_recv, cam_base=cam_end - cam_size, field_off=field_off, recv_bytes=int(cam_end[:, -1].max()),
                first_row=S[:me].sum(0), grad_row=grad_row, grad_rows_max=int(per_src.sum(1).max()))


class PeerArena:
    """Symmetric-memory receive arena (forward rows) and gradient staging buffer (backward rows) of one group."""

    def __init__(self, group, device):
        import torch.distributed._symmetric_memory as symm

        self._symm = symm
        self.group = group if group is not None else dist.group.WORLD
        self.dev = device
        # Two receive arenas, used by alternate steps: while a rank still reads what step s delivered (its render and
        # backward passes), a peer that is already in step s + 1 writes into the other one; a peer can only reach
        # step s + 2 through the "rows have landed" barrier of step s + 1, which this rank joins after it has queued
        # everything of step s.  So no barrier is needed before the stores of a step.
        self._recv = [None, None]
        self._recv_hdl = [None, None]
        self.grad = self.grad_hdl = None
        self.ws, self.me = dist.get_world_size(self.group), dist.get_rank(self.group)
        # flag words for the stream-ordered barrier: zeroed before any rank can signal
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self.flags_hdl = symm.rendezvous(self.flags, self.group)
        dist.barrier(group=self.group)
        # One exchange = one step of the arena.  The two barriers of step s carry the epochs 3s+2 (forward rows have
        # landed) and 3s+3 (gradient rows have landed): absolute numbers, so a rank whose backward pass did not run
        # (nothing of what it received reached its loss) cannot fall one barrier behind the others for the rest of
        # the run.
        self.step = 0
        self.last_grad_step = -1       # step of the latest exchange that built an autograd node
        self._flag_ptrs = (C.c_void_p * self.ws)(*[int(p) for p in self.flags_hdl.buffer_ptrs])

    def _alloc(self, nbytes):
        nbytes = _align_up(int(nbytes * 1.25) + (1 << 20), 2 << 20)
        t = self._symm.empty(nbytes, dtype=torch.uint8, device=self.dev)
        return t, self._symm.rendezvous(t, self.group)

    @property
    def recv(self):
        return self._recv[self.step & 1]

    @property
    def recv_hdl(self):
        return self._recv_hdl[self.step & 1]

    def ensure(self, recv_bytes, grad_bytes):
        """Grow (collectively: every rank passes the same numbers) so that every rank's arenas hold these sizes."""
        for p in (0, 1):
            if self._recv[p] is None or self._recv[p].numel() < recv_bytes:
                self._recv[p], self._recv_hdl[p] = self._alloc(recv_bytes)
        if grad_bytes and (self.grad is None or self.grad.numel() < grad_bytes):
            self.grad, self.grad_hdl = self._alloc(grad_bytes)

    def begin_step(self):
        """Start the next exchange: it uses the other receive arena.  The tensors the exchange before the previous one
        returned are dead from here on."""
        self.step += 1

    def barrier(self, phase):
        """Stream-ordered barrier over the group: work queued before it on every rank is complete after it."""
        from diff_gaussian_rasterization import _lib

        epoch = (3 * self.step + phase) & 0xFFFFFFFF
        _lib.check(_lib.lib().cgx_peer_barrier(self.ws, self.me, self._flag_ptrs, epoch, _lib.current_stream_ptr()),
                   "cgx_peer_barrier")


_arenas = {}


def _arena_for(group, device):
    key = (id(group), device)
    if key not in _arenas:
        _arenas[key] = PeerArena(group, device)
    return _arenas[key]


def _camera_order(strategies, me, ws):
    """The order in which a rank's pack launch works through the cameras: first those the rank after it renders,
    its own last, so that at any time the ranks store into different peers (all of them sending camera 0's rows
    first would queue on the links of the rank that renders camera 0)."""
    return sorted(range(len(strategies)), key=lambda k: ((strategies[k].gpu_ids[0] - me - 1) % ws, k))


def _destination_rows(field_ptr, first_row, cam, dst, planes):
    """Rows of struct cgx_peer_camera_dst for the (camera, rendering rank) pairs (cam[e], dst[e]): the addresses of
    the camera's tensors in that rank's arena (field_ptr[rank, camera, field]) and the first row this rank writes."""
    rows = np.zeros((cam.size, 10), dtype=np.uint64)
    rows[:, [0, 1, 2, 9, 6, 7] if planes else list(range(8))] = field_ptr[dst, cam, :]
    rows[:, 8] = first_row[dst, cam]
    return rows


def _p2p_forward(plan):
    """Pack this rank's rows into the peers' receive arenas, wait until every rank's rows have landed, and return
    (per-camera views of this rank's arena, the non-differentiable ones among them)."""
    be, arena = plan["backend"], plan["arena"]
    me = plan["me"]
    bsz = len(plan["strategies"])
    planes = plan["planes"]
    peer_base = np.array([int(p) for p in arena.recv_hdl.buffer_ptrs], dtype=np.int64)
    # address of field f of camera k in rank j's arena, and the first row this rank writes there
    field_ptr = peer_base[:, None, None] + plan["cam_base"][:, :, None] + plan["field_off"]      # (ws, bsz, F)
    # (the barrier "every rank is done with the previous contents of the arenas" was queued by the caller,
    # behind the size read-back)
    prep = plan.get("prepared")
    if prep is not None:
        # destination rows of every (camera, rendering rank) pair at once, in the prepared camera order
        cam, dst = prep["entry_cam"], prep["entry_dst"]
        rows = _destination_rows(field_ptr, plan["first_row"], cam, dst, planes)
        be.pack_p2p_prepared(prep, rows, plan["send_off"][dst, cam], plan["send_index"])
    else:
        cameras = []
        for k in range(bsz):
            ids = plan["strategies"][k].gpu_ids
            table = np.zeros((len(ids), 10), dtype=np.uint64)      # rows = struct cgx_peer_camera_dst
            if planes:
                table[:, [0, 1, 2, 9, 6, 7]] = field_ptr[ids, k, :]
            else:
                table[:, :8] = field_ptr[ids, k, :]
            table[:, 8] = plan["first_row"][ids, k]
            cameras.append(dict(params=plan["params"][k], bounds=plan["bounds"][k], H=plan["hw"][k][0],
                                W=plan["hw"][k][1], avoid=plan["avoid"][k], dst_table=table,
                                row_offsets=plan["send_off"][ids, k], workspace=plan["scratch"][k]))
        cameras = [cameras[k] for k in _camera_order(plan["strategies"], me, plan["ws"])]
        if hasattr(be, "pack_p2p_batched"):
            be.pack_p2p_batched(cameras, plan["send_index"])
        else:
            for c in cameras:
                be.pack_p2p(c["params"], c["bounds"], c["H"], c["W"], c["avoid"], c["dst_table"], c["row_offsets"],
                            plan["send_index"], c["workspace"])
    arena.barrier(2)                      # every rank's rows have landed
    outs, nondiff = [], []
    f32 = arena.recv.view(torch.float32)
    i32 = arena.recv.view(torch.int32)
    words = ((plan["cam_base"][me][:, None] + plan["field_off"][me]) // 4).tolist()   # offsets in 4-byte words
    n_mine = plan["n_recv"][me].tolist()
    for k in range(bsz):
        n, w = n_mine[k], words[k]
        m2 = f32[w[0]: w[0] + 2 * n].view(n, 2)
        rgb = f32[w[1]: w[1] + 3 * n].view(n, 3)
        co = f32[w[2]: w[2] + 4 * n].view(n, 4)
        if planes:
            am = f32[w[3]: w[3] + 5 * n].view(n, 5)
            rad = i32[w[4]: w[4] + n]
            dep = f32[w[5]: w[5] + n]
            outs += [m2, rgb, co, rad, dep, am]
        else:
            m3 = f32[w[3]: w[3] + 3 * n].view(n, 3)
            sc = f32[w[4]: w[4] + 3 * n].view(n, 3)
            rot = f32[w[5]: w[5] + 4 * n].view(n, 4)
            rad = i32[w[6]: w[6] + n]
            dep = f32[w[7]: w[7] + n]
            outs += [m2, rgb, co, rad, dep, m3, sc, rot]
        nondiff += [rad, dep]
    return outs, nondiff


def _p2p_send_gradients(plan, gouts):
    """Reverse leg: store the cotangent rows of what this rank received into their owners' staging buffers and wait
    until every rank's rows have landed.  Returns the rows this rank owns, (n_send, grad_cols), in send order."""
    be, arena = plan["backend"], plan["arena"]
    me, S = plan["me"], plan["S"]
    dev = arena.dev
    bsz = len(plan["strategies"])
    ncols = plan["grad_cols"]
    planes = plan["planes"]
    n_out = 6 if planes else 8
    if arena.last_grad_step != plan["arena_step"] or arena.step - plan["arena_step"] > 1:
        raise RuntimeError(
            "cgx.exchange: the backward pass of a peer-to-peer exchange ran too late: another exchange with a "
            "graph, or two exchanges without one, have used the same group since its forward pass, and the "
            "tensors it returned (views of a receive arena) or its gradient staging buffer were overwritten.  "
            "Keep one differentiable exchange in flight per group (at most one forward-only exchange may come "
            "between its forward and backward passes), or use transport='collective'")
    owner_base = np.array([int(p) for p in arena.grad_hdl.buffer_ptrs], dtype=np.int64)
    # segment (source i -> me, camera k) sits at row grad_row[i, k] of rank i's send order
    seg_ptr = owner_base[:, None] + plan["grad_row"] * (ncols * 4)                                # (ws, bsz)
    for k in range(bsz):
        counts = S[:, me, k]
        if not counts.any():
            continue                      # camera not rendered here: no gradient rows to return
        g = gouts[n_out * k: n_out * k + n_out]
        n = int(plan["n_recv"][me, k])
        if planes:                        # the (n,5) plane-descriptor cotangent rides in the means3D slot
            cot = _dense_cotangents((g[0], g[1], g[2], None, None, None, None, None), n, dev)[:3] + \
                (g[5] if g[5] is not None else torch.zeros(n, 5, device=dev), None, None)
        else:
            cot = _dense_cotangents(g, n, dev)
        # every rank starts with the rows of the rank after it: the ranks' stores go to different peers at any time
        be.pack_grad_rows_to(seg_ptr[:, k].tolist(), counts.tolist(), ncols, cot, first_segment=me + 1)
    arena.barrier(3)                      # every rank's gradient rows have landed in their owners' buffers
    n_send = plan["n_send"]
    return arena.grad[: n_send * ncols * 4].view(torch.float32).view(n_send, ncols)


class _GaussianExchangeP2P(torch.autograd.Function):
    """Same contract as _GaussianExchange, transport by direct stores into peer memory."""

    @staticmethod
    def forward(ctx, plan, *flat):
        outs, nondiff = _p2p_forward(plan)
        ctx.plan = plan
        ctx.shapes = [t.shape for t in flat]
        ctx.mark_non_differentiable(*nondiff)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *gouts):
        plan = ctx.plan
        be, dev, planes, ncols = plan["backend"], plan["arena"].dev, plan["planes"], plan["grad_cols"]
        n_in = 4 if planes else 6
        grad_send = _p2p_send_gradients(plan, gouts)
        grads = []
        for k, per_dst in enumerate(plan["send_ranges"]):
            need = ctx.needs_input_grad[1 + n_in * k: 1 + n_in * k + n_in]
            shapes = ctx.shapes[n_in * k: n_in * k + n_in]
            gk = [torch.zeros(s, dtype=torch.float32, device=dev) if nd else None for s, nd in zip(shapes, need)]
            for c in (0, 2):                  # the scatter kernel always writes means2D and conic_opacity
                if gk[c] is None:
                    gk[c] = torch.zeros(shapes[c], dtype=torch.float32, device=dev)
            be.unpack_grad_add_cols(grad_send, plan["send_index"], per_dst, ncols,
                                    gk + [None, None] if planes else gk)
            grads += [g if nd else None for g, nd in zip(gk, need)]
        return (None,) + tuple(grads)


class _RowSegment(C.Structure):
    _fields_ = [("start", C.c_longlong), ("count", C.c_longlong), ("camera", C.c_int), ("reserved", C.c_int)]


class _OwnerExchangeP2P(torch.autograd.Function):
    """The peer-to-peer exchange of plane-descriptor records with the owner's preprocess backward folded into its
    backward pass: inputs are the four parameter tensors the camera-batched preprocess read (its outputs enter the
    exchange detached), outputs are the received per-camera tensors.  In the backward the gradient rows that come
    back are consumed where they land (`cgx_preprocess_bwd_rows`): no dense per-camera cotangent arrays, no
    scatter, and only pairs that were visible somewhere do any work."""

    @staticmethod
    def forward(ctx, plan, owner, means3D, scales, rotations, opacities):
        outs, nondiff = _p2p_forward(plan)
        ctx.plan, ctx.owner = plan, owner
        ctx.save_for_backward(means3D, scales, rotations)
        ctx.op_shape = opacities.shape
        ctx.mark_non_differentiable(*nondiff)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *gouts):
        from diff_gaussian_rasterization import _C, _lib

        from .batched import _cams, _ptrs

        plan, owner = ctx.plan, ctx.owner
        means3D, scales, rotations = ctx.saved_tensors
        means3D, scales, rotations = means3D.contiguous(), scales.contiguous(), rotations.contiguous()
        rows = _p2p_send_gradients(plan, gouts)
        settings = owner["settings"]
        P, dev, ncols = means3D.shape[0], means3D.device, plan["grad_cols"]
        segs = [(a, b - a, k) for k, per_dst in enumerate(plan["send_ranges"]) for a, b in per_dst if b > a]
        arr = (_RowSegment * max(len(segs), 1))()
        for e, (a, n, k) in zip(arr, segs):
            e.start, e.count, e.camera = a, n, k
        d_means = torch.empty(P, 3, device=dev)
        d_scales = torch.empty(P, 3, device=dev)
        d_rot = torch.empty(P, 4, device=dev)
        d_op = torch.empty(ctx.op_shape, device=dev)
        if P:
            l = _lib.lib()
            cams, keep = _cams(settings)
            campos = [rs.campos.contiguous() for rs in settings]
            work = torch.empty(l.cgx_preprocess_bwd_rows_workspace_bytes(P), dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                _C._call("cgx_preprocess_bwd_rows", l.cgx_preprocess_bwd_rows, P, len(segs), arr, ncols,
                         C.c_void_p(rows.data_ptr()), C.c_void_p(plan["send_index"].data_ptr()),
                         C.c_void_p(means3D.data_ptr()), C.c_void_p(scales.data_ptr()),
                         float(settings[0].scale_modifier), C.c_void_p(rotations.data_ptr()), len(settings), cams,
                         _ptrs(campos), C.c_void_p(work.data_ptr()), work.numel(), C.c_void_p(d_means.data_ptr()),
                         C.c_void_p(d_scales.data_ptr()), C.c_void_p(d_rot.data_ptr()), C.c_void_p(d_op.data_ptr()),
                         _lib.current_stream_ptr(), info=dict(P=P, rows=rows.shape[0], ncols=ncols))
            pipeline = owner.get("pipeline")
            if pipeline is not None and pipeline.done is not None:
                for i, (lo, hi) in enumerate(pipeline.bounds):
                    pipeline.done(i, lo, hi, (d_means, d_scales, d_rot, d_op))
        return None, None, d_means, d_scales, d_rot, d_op


def _pick_transport(transport, group, dev, backend):
    if transport is not None:
        return transport
    import os

    if os.environ.get("CGX_EXCHANGE", "").lower() in ("collective", "nccl"):
        return "collective"
    if dev.type == "cuda" and dist.get_backend(group) == "nccl" and hasattr(backend, "pack_p2p"):
        return "p2p"
    return "collective"


def all_to_all_communication_final(batched_rasterizers, batched_screenspace_params, batched_cuda_args,
                                   batched_strategies, group=None, backend=None, transport=None, piggyback=None,
                                   planes=False, owner=None):
    """See module docstring.  ``batched_screenspace_params[k]`` =
    (means2D, rgb, conic_opacity, radii, depths, means3D, scales, rotation) of camera k on this rank.

    Returns the reference's tuple: per-camera lists of means2D, rgb, conic_opacity, radii (int32), depths, means3D,
    scales, rotations (redistributed), then the size table [src][dst][cam] and the rows sent per destination and
    camera (the reference returns index tensors there; here the source indices stay on the device in one packed
    tensor, returned next), and a dict of transfer statistics.

    ``piggyback``: optional list of floats (same length on every rank) that rides on the size-table all-gather;
    every rank's values come back as ``stats["piggyback"][rank]``.  The balancer's render times travel this way
    instead of in a collective (and a host synchronisation) of their own.

    ``planes=True`` (peer-to-peer transport only): ``batched_screenspace_params[k]`` = (means2D, rgb,
    conic_opacity, radii, depths, all_map) with the camera's plane descriptors already computed by the owner
    (`cgx.batched.preprocess_gaussians_batched(planes=True)`).  The descriptors travel instead of the 3-D
    parameters they would be rebuilt from on the receiver (16 floats per row instead of 21, 14 gradient columns
    back instead of 19); the sixth returned list then holds ``all_map`` per camera and the last two are None.

    ``owner`` (with ``planes=True``): ``dict(params=(means3D, scales, rotations, opacities), settings=[raster settings
    of every camera], pipeline=None)`` of the camera-batched preprocess call that produced the (then detached)
    screen-space tensors.  The exchange becomes the one autograd node between the parameters and the received
    tensors, and its backward pass runs the owner's preprocess backward straight over the gradient rows that come
    back (`cgx_preprocess_bwd_rows`).  The owner-side screen-space tensors get no ``.grad`` in this form."""
    backend = backend or default_backend()
    ws, me = _world(group)
    bsz = len(batched_rasterizers)
    dev = batched_screenspace_params[0][0].device

    # ---- 1. counts: one kernel pair per camera, results land in one (bsz, ws) table, ONE host read
    n_extra = len(piggyback) if piggyback is not None else 0
    table_dev = torch.zeros(bsz * ws + n_extra, dtype=torch.int32, device=dev)
    counts_dev = table_dev[: bsz * ws].view(bsz, ws)
    scratch, bounds, jobs, scattered = [], [], [], []
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
        jobs.append((means2D.detach().contiguous(), radii.contiguous(), tb, rs.image_height, rs.image_width,
                     batched_cuda_args[k]["avoid_pixel_all2all"], c, wspace))
        if not contiguous_ranks:
            scattered.append((k, strat.gpu_ids, c))
        scratch.append(wspace)
        bounds.append(tb)
    if hasattr(backend, "count_batched"):
        backend.count_batched(jobs)              # every camera's counts in two launches
    else:
        for job in jobs:
            backend.count(*job)
    for k, ids, c in scattered:
        counts_dev[k, torch.as_tensor(ids, device=dev, dtype=torch.long)] = c
    if dist.get_backend(group) != "nccl":
        table_dev = table_dev.cpu()
    transport = _pick_transport(transport, group, dev, backend)
    if planes and transport != "p2p":
        raise RuntimeError("the plane-descriptor record form needs the peer-to-peer transport")
    arena = _arena_for(group, dev) if transport == "p2p" else None
    # the barrier "every rank is done with the previous contents of the arenas" does not depend on the sizes: it is
    # queued behind the size read-back and runs while the host lays out the exchange
    # While the host waits for the size table it prepares everything of the pack launch that does not depend on it
    # (and the flat argument lists): what is left between the table's arrival and the launch is a few array operations.
    flat = []
    for k in range(bsz):
        if planes:
            m2, rgb, co, radii, depths, am = batched_screenspace_params[k]
            flat += [m2, rgb, co, am]
        else:
            m2, rgb, co, radii, depths, m3, sc, rot = batched_screenspace_params[k]
            flat += [m2, rgb, co, m3, sc, rot]
    early = {}

    def while_waiting():
        arena.begin_step()
        early["params"] = [tuple(t.detach() for t in p) for p in batched_screenspace_params]
        early["hw"] = [(r.raster_settings.image_height, r.raster_settings.image_width) for r in batched_rasterizers]
        early["avoid"] = [a["avoid_pixel_all2all"] for a in batched_cuda_args]
        if hasattr(backend, "prepare_pack_p2p"):
            order = _camera_order(batched_strategies, me, ws)
            cams = [dict(params=early["params"][k], bounds=bounds[k], H=early["hw"][k][0], W=early["hw"][k][1],
                         avoid=early["avoid"][k], workspace=scratch[k]) for k in range(bsz)]
            prep = backend.prepare_pack_p2p(cams, order)
            ids = [batched_strategies[k].gpu_ids for k in order]
            prep["entry_cam"] = np.repeat(np.asarray(order, dtype=np.int64), [len(i) for i in ids])
            prep["entry_dst"] = np.concatenate([np.asarray(i, dtype=np.int64) for i in ids])
            early["prepared"] = prep

    gathered, extra = _gather_table(table_dev, bsz * ws, piggyback, group, ws,
                                    overlap=while_waiting if arena is not None else None)
    S = np.ascontiguousarray(gathered.reshape(ws, bsz, ws).transpose(0, 2, 1))     # [src][dst][cam]
    my = S[me]                                                       # [dst][cam]

    # ---- 2. send order: destination major, camera minor
    send_splits = my.sum(1).tolist()
    recv_splits = S[:, me, :].sum(1).tolist()
    n_send = int(my.sum())
    ends = np.cumsum(my.reshape(-1))
    send_off = (ends - my.reshape(-1)).reshape(ws, bsz)              # first send row of (destination, camera)
    send_index = torch.empty(n_send, dtype=torch.int32, device=dev)

    def bookkeeping():
        """What the caller and the backward pass want to know; nothing the forward launches need."""
        send_ranges = [[(int(send_off[j, k]), int(send_off[j, k] + my[j, k])) for j in batched_strategies[k].gpu_ids]
                       for k in range(bsz)]
        self_rows = int(my[me].sum())
        stats = {"rows_sent": n_send, "rows_received": sum(recv_splits), "rows_to_self": self_rows,
                 "bytes_sent_fwd": (n_send - self_rows) * REC * 4, "bytes_sent_bwd": (n_send - self_rows) * REC_DIFF * 4,
                 "piggyback": extra, "transport": transport}
        return send_ranges, S.tolist(), my.tolist(), stats

    if transport == "p2p":
        lay = p2p_layout(S, me, _CAM_FIELDS_PLANES if planes else _CAM_FIELDS)
        n_recv, field_off, grad_row = lay["n_recv"], lay["field_off"], lay["grad_row"]
        arena.ensure(lay["recv_bytes"], lay["grad_rows_max"] * REC_DIFF * 4)
        # gradient rows carry 19 columns only when some rank needs gradients for the 3-D parameters through the
        # exchange; every rank runs the same model code, so this is the same decision everywhere
        if planes:
            grad_cols = 14 if owner is not None or any(flat[4 * k + 3].requires_grad for k in range(bsz)) else 9
        else:
            grad_cols = REC_DIFF if any(flat[6 * k + c].requires_grad for k in range(bsz) for c in (3, 4, 5)) else 9
        # send_ranges (read by the backward pass only) joins the plan after the launches have been queued
        plan = dict(backend=backend, arena=arena, arena_step=arena.step, me=me, ws=ws, S=S, strategies=batched_strategies,
                    grad_cols=grad_cols, planes=planes, n_recv=n_recv, cam_base=lay["cam_base"], field_off=field_off,
                    first_row=lay["first_row"], grad_row=grad_row, bounds=bounds, scratch=scratch,
                    send_index=send_index, send_off=send_off, n_send=n_send, params=early["params"], hw=early["hw"],
                    avoid=early["avoid"], prepared=early.get("prepared"))
        if owner is not None:
            if not planes:
                raise RuntimeError("owner= needs the plane-descriptor record form (planes=True)")
            if torch.is_grad_enabled() and any(t.requires_grad for t in owner["params"]):
                arena.last_grad_step = arena.step
            outs = _OwnerExchangeP2P.apply(plan, owner, *owner["params"])
        else:
            if torch.is_grad_enabled() and any(t.requires_grad for t in flat):
                arena.last_grad_step = arena.step
            outs = _GaussianExchangeP2P.apply(plan, *flat)
        plan["send_ranges"], sizes_list, sent_counts, stats = bookkeeping()
        self_rows = stats["rows_to_self"]
        if planes:
            stats["bytes_sent_fwd"] = (n_send - self_rows) * 16 * 4
        stats["bytes_sent_bwd"] = (n_send - self_rows) * grad_cols * 4
        if planes:
            out = [[outs[6 * k + c] for k in range(bsz)] for c in range(6)] + [None, None]
        else:
            out = [[outs[8 * k + c] for k in range(bsz)] for c in range(8)]
        return (*out, sizes_list, sent_counts, send_index, stats)

    # ---- 2b. collective transport: send buffer packed by one kernel per camera
    send_ranges, sizes_list, sent_counts, stats = bookkeeping()
    send = torch.empty(n_send, REC_DIFF, dtype=torch.float32, device=dev)
    send_aux = torch.empty(n_send, REC - REC_DIFF, dtype=torch.float32, device=dev)
    for k in range(bsz):
        params = tuple(t.detach() for t in batched_screenspace_params[k])
        rs = batched_rasterizers[k].raster_settings
        backend.pack(params, bounds[k], rs.image_height, rs.image_width, batched_cuda_args[k]["avoid_pixel_all2all"],
                     [a for a, _ in send_ranges[k]], send, send_aux, send_index, scratch[k])

    # ---- 3. receive layout: source major, camera minor -> per camera one segment per source
    from_src = S[:, me, :]                                            # [src][cam]
    ends = np.cumsum(from_src.reshape(-1))
    recv_off = (ends - from_src.reshape(-1)).reshape(ws, bsz)
    recv_segments = [[(int(recv_off[i, k]), int(from_src[i, k])) for i in range(ws)] for k in range(bsz)]

    plan = dict(backend=backend, group=group, send=send, send_aux=send_aux, send_index=send_index,
                send_splits=send_splits, recv_splits=recv_splits, send_ranges=send_ranges,
                recv_segments=recv_segments)
    outs = _GaussianExchange.apply(plan, *flat)
    out = [[outs[8 * k + c] for k in range(bsz)] for c in range(8)]
    return (*out, sizes_list, sent_counts, send_index, stats)


# ----------------------------------------------------------------------------------------------------------------
# Row redistribution by a destination vector (the reference's anchor redistribution)
def _as_words(t):
    """A (N, ...) tensor as rows of 4-byte words: (tensor to move, words per row, how to turn received words back).
    Rows whose byte size is not a multiple of 4 (bool / int8 / int16 tags) travel widened to int32."""
    n = t.shape[0]
    row_bytes = (t.numel() // n if n else int(np.prod(t.shape[1:], dtype=np.int64))) * t.element_size()
    if t.dtype == torch.bool or row_bytes % 4:
        wide = t.to(torch.int32).contiguous()
        return wide, int(np.prod(t.shape[1:], dtype=np.int64)), (torch.int32, t.dtype)
    return t.contiguous(), row_bytes // 4, (t.dtype, t.dtype)


class _CudaRowsBackend:
    """Counting / packing / splitting of redistributed rows on the GPU through the C ABI."""

    def __init__(self):
        from diff_gaussian_rasterization import _lib

        self._lib, self.l = _lib, _lib.lib()

    def count(self, dest32, ws):
        n, dev = dest32.numel(), dest32.device
        if not dest32.is_cuda:
            raise RuntimeError("cgx.exchange: the row packing backend needs CUDA tensors (no CPU path)")
        counts = torch.empty(ws + 1, dtype=torch.int32, device=dev)
        work = torch.empty(self.l.cgx_rows_workspace_bytes(n, ws), dtype=torch.uint8, device=dev)
        self._lib.check(self.l.cgx_rows_dest_count(n, ws, C.c_void_p(dest32.data_ptr()), C.c_void_p(counts.data_ptr()),
                                                   C.c_void_p(work.data_ptr()), work.numel(),
                                                   self._lib.current_stream_ptr()), "cgx_rows_dest_count")
        return counts, work

    def pack(self, dest32, ws, tensors, words, dst_base, first_row, work):
        """dst_base: the (rows, row_words) int32 send buffer every destination's segment lives in, or one device
        address per destination (a peer's arena)."""
        n, k = dest32.numel(), len(tensors)
        if isinstance(dst_base, torch.Tensor):
            dst_base = [dst_base.data_ptr()] * ws
        ptrs = (C.c_void_p * k)(*[t.data_ptr() for t in tensors])
        w = (C.c_int32 * k)(*words)
        base = (C.c_void_p * ws)(*[int(b) for b in dst_base])
        first = (C.c_int64 * ws)(*[int(f) for f in first_row])
        self._lib.check(self.l.cgx_rows_pack(n, ws, C.c_void_p(dest32.data_ptr()), k, ptrs, w, base, first,
                                             C.c_void_p(work.data_ptr()), self._lib.current_stream_ptr()),
                        "cgx_rows_pack")

    def unpack(self, rows_ptr, n, outs, words):
        k = len(outs)
        ptrs = (C.c_void_p * k)(*[t.data_ptr() for t in outs])
        w = (C.c_int32 * k)(*words)
        if isinstance(rows_ptr, torch.Tensor):
            rows_ptr = rows_ptr.data_ptr()
        self._lib.check(self.l.cgx_rows_unpack(n, C.c_void_p(int(rows_ptr)), k, ptrs, w,
                                               self._lib.current_stream_ptr()), "cgx_rows_unpack")


_rows_backend = None


def redistribute_rows(tensors, destination, group=None, backend=None, transport=None):
    """Move row i of every tensor to rank ``destination[i]``: the reference's anchor redistribution
    (scene/gaussian_model.py:1485-1558 ``all2all_gaussian_state`` applied to every parameter, both Adam moments and
    the level tags by ``redistribute_gaussians`` :1683-1764 — about eighteen list all-to-alls) as ONE exchange.

    ``tensors``: list of tensors with the same number of rows N (any shape behind the first dimension, any dtype);
    ``destination``: (N,) integer tensor of ranks.  Returns ``(new_tensors, i2j_send_size)``: every tensor with the
    rows this rank received — sources in ascending rank order, within a source ascending local index, exactly the
    reference's ``torch.cat(state_from_gpuj)`` — and the (ws, ws) table of rows sent from i to j as nested lists.

    One counting kernel, one host read of the gathered counts (the reference does the same read), one packing kernel
    for all tensors (a travelling row is the concatenation of the tensors' rows), then either one
    ``all_to_all_single`` (``transport="collective"``, any backend) or direct stores into the peers' symmetric-memory
    arenas bracketed by the bounded device barrier (``"p2p"``, the default inside an NCCL group), one splitting kernel."""
    global _rows_backend
    ws, me = _world(group)
    if backend is None:
        if _rows_backend is None:
            _rows_backend = _CudaRowsBackend()
        backend = _rows_backend
    n = destination.numel()
    dev = destination.device
    for t in tensors:
        if t.shape[0] != n:
            raise RuntimeError("redistribute_rows: every tensor needs one row per entry of `destination`")
    dest32 = destination.to(torch.int32).contiguous()
    moved = [_as_words(t.detach()) for t in tensors]
    words = [m[1] for m in moved]
    row_words = sum(words)

    counts, work = backend.count(dest32, ws)
    table = counts if dist.get_backend(group) == "nccl" else counts.cpu()
    out = torch.empty(ws * (ws + 1), dtype=torch.int32, device=table.device)
    dist.all_gather_into_tensor(out, table, group=group)
    host = out.cpu().numpy().reshape(ws, ws + 1).astype(np.int64)          # the one host synchronisation
    if host[:, ws].any():
        raise RuntimeError("redistribute_rows: a destination outside [0, world_size)")
    S = host[:, :ws]                                                        # S[i][j] = rows i sends to j
    n_recv, n_send = int(S[:, me].sum()), int(S[me].sum())
    if n_send != n:
        raise RuntimeError("redistribute_rows: counted rows do not add up to the number of rows")

    if transport is None:
        import os

        forced = os.environ.get("CGX_EXCHANGE", "").lower() in ("collective", "nccl")
        transport = "p2p" if (not forced and dev.type == "cuda" and dist.get_backend(group) == "nccl") else "collective"
    if transport == "p2p":
        arena = _arena_for(group, dev)
        arena.ensure(int(S.sum(0).max()) * row_words * 4, 0)
        arena.begin_step()
        bases = [int(p) for p in arena.recv_hdl.buffer_ptrs]
        if n:
            backend.pack(dest32, ws, [m[0] for m in moved], words, bases, S[:me].sum(0).tolist(), work)
        arena.barrier(2)                       # every rank's rows have landed
        rows_ptr = arena.recv.data_ptr()
        keep = arena.recv
    else:
        send = torch.empty(max(n_send, 1), max(row_words, 1), dtype=torch.int32, device=dev)
        first = (np.cumsum(S[me]) - S[me]).tolist()
        if n:
            backend.pack(dest32, ws, [m[0] for m in moved], words, send, first, work)
        recv = torch.empty(max(n_recv, 1), max(row_words, 1), dtype=torch.int32, device=dev)
        dist.all_to_all_single(recv[:n_recv], send[:n_send], output_split_sizes=S[:, me].tolist(),
                               input_split_sizes=S[me].tolist(), group=group)
        rows_ptr, keep = recv.data_ptr(), recv
    outs = [torch.empty((n_recv,) + tuple(t.shape[1:]), dtype=m[2][0], device=dev) for t, m in zip(tensors, moved)]
    if n_recv:
        backend.unpack(rows_ptr if transport == "p2p" else keep, n_recv, outs, words)
    del keep
    outs = [o if m[2][0] == m[2][1] else o.to(m[2][1]) for o, m in zip(outs, moved)]
    return outs, S.tolist()
