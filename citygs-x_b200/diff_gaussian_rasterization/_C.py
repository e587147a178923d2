"""Drop-in for the reference's compiled ``diff_gaussian_rasterization._C`` module.

Same 14 entry points, argument order, return tuples and error behaviour as the pybind module of the
reference (RAST/ext.cpp:17-34, signatures RAST/rasterize_points.h), implemented as thin PyTorch host code
(allocation, stream plumbing) over the hand-written sm_100a kernels behind the C ABI of
include/cgx_raster.h.  No CPU path: tensors must live on a CUDA device.

Scratch ("geomBuffer", "binningBuffer", "imgBuffer") is returned as uint8 tensors carved with the
reference's own layout rules (128-byte aligned sub-arrays in the same order,
RAST/cuda_rasterizer/rasterizer_impl.cu:161-205, rasterizer_impl.h:21-27), so tooling that decodes the
reference's buffers (point_list, sorted keys, ranges, final T, n_contrib) decodes these as well.  The
geometry buffer additionally carries the packed 64-byte per-Gaussian records the blending kernels stage.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import check

BLOCK_X, BLOCK_Y, ONE_DIM_BLOCK_SIZE = 16, 16, 256
NUM_CHANNELS, NUM_ALL_MAP = 3, 5


# Optional per-stage profiling: when PROFILE is a list, every C-ABI call is bracketed by two CUDA events on the
# current stream and (stage, start, end, info) is appended; the owner resolves the events after a synchronise.
PROFILE = None


def _call(stage, fn, *a, info=None):
    prof = PROFILE
    if prof is None:
        check(fn(*a), stage)
        return
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    check(fn(*a), stage)
    e1.record()
    prof.append((stage, e0, e1, info))


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return _lib.current_stream_ptr()


def _cuda_f32(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this rasterizer has no CPU path)")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32")
    return t.contiguous()


def _cuda_any(t, name):
    """Any-dtype tensor that a kernel will dereference: must live on a CUDA device, returned contiguous."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this rasterizer has no CPU path)")
    return t.contiguous()


def _align(n, a=128):
    return (n + a - 1) // a * a


_ITEMSIZE = {torch.uint8: 1, torch.bool: 1, torch.int32: 4, torch.float32: 4, torch.int64: 8}


class _Carver:
    """Sub-arrays of one uint8 tensor, each starting on a 128-byte boundary, in declaration order."""

    def __init__(self):
        self.items, self.size = [], 0

    def add(self, name, dtype, count):
        off = _align(self.size)
        nbytes = count * _ITEMSIZE[dtype]
        self.items.append((name, dtype, nbytes, off))
        self.size = off + nbytes
        return self

    def total(self):
        return self.size + 128

    def views(self, buf):
        return {name: buf[off:off + nbytes].view(dtype) for name, dtype, nbytes, off in self.items}


import functools


@functools.lru_cache(maxsize=256)
def geometry_layout(P):
    l = _lib.lib()
    return (_Carver().add("tiles_touched", torch.int32, P)
            .add("scanning_space", torch.uint8, l.cgx_bin_workspace_bytes(P))
            .add("point_offsets", torch.int32, P)
            .add("num_rendered", torch.int32, 32)
            .add("records", torch.uint8, l.cgx_render_records_bytes(P)))


@functools.lru_cache(maxsize=256)
def binning_layout(R):
    l = _lib.lib()
    return (_Carver().add("point_list", torch.int32, R)
            .add("point_list_unsorted", torch.int32, R)
            .add("point_list_keys", torch.int64, R)
            .add("point_list_keys_unsorted", torch.int64, R)
            .add("list_sorting_space", torch.uint8, l.cgx_sort_workspace_bytes(R)))


@functools.lru_cache(maxsize=64)
def image_layout(N, T):
    return (_Carver().add("accum_alpha", torch.float32, N)
            .add("n_contrib", torch.int32, N)
            .add("n_contrib2loss", torch.int32, N)
            .add("ranges", torch.int32, 2 * T))


# ----------------------------------------------------------------------------- the 14 entry points
def get_block_XY():
    return (BLOCK_X, BLOCK_Y, ONE_DIM_BLOCK_SIZE)


def mark_visible(means3D, viewmatrix, projmatrix):
    means3D = _cuda_f32(means3D, "means3D")
    P = means3D.shape[0]
    present = torch.empty(P, dtype=torch.bool, device=means3D.device)
    if P:
        with torch.cuda.device(means3D.device):
            _call("cgx_mark_visible", _lib.lib().cgx_mark_visible, P, _ptr(means3D), _ptr(_cuda_f32(viewmatrix, "viewmatrix")),
                                              _ptr(present), _stream())
    return present


def preprocess_gaussians(means3D, scales, rotations, sh, opacity, scale_modifier, viewmatrix, projmatrix,
                         tan_fovx, tan_fovy, image_height, image_width, degree, campos, prefiltered, debug, args):
    if means3D.ndim != 2 or means3D.shape[1] != 3:
        raise RuntimeError("means3D must have dimensions (num_points, 3)")
    means3D = _cuda_f32(means3D, "means3D")
    P, dev = means3D.shape[0], means3D.device
    means2D = torch.empty(P, 2, dtype=torch.float32, device=dev)
    depths = torch.empty(P, dtype=torch.float32, device=dev)
    radii = torch.empty(P, dtype=torch.int32, device=dev)
    cov3D = torch.empty(P, 6, dtype=torch.float32, device=dev)
    conic_opacity = torch.empty(P, 4, dtype=torch.float32, device=dev)
    # SH evaluation is compiled out upstream: rgb stays zero and nothing is ever clamped
    rgb = torch.zeros(P, 3, dtype=torch.float32, device=dev)
    clamped = torch.zeros(P, 3, dtype=torch.bool, device=dev)
    if P:
        with torch.cuda.device(dev):
            _call("cgx_preprocess_fwd", _lib.lib().cgx_preprocess_fwd, 
                P, _ptr(means3D), _ptr(_cuda_f32(scales, "scales")), float(scale_modifier),
                _ptr(_cuda_f32(rotations, "rotations")), _ptr(_cuda_f32(opacity, "opacity")),
                _ptr(_cuda_f32(viewmatrix, "viewmatrix")), _ptr(_cuda_f32(projmatrix, "projmatrix")),
                int(image_width), int(image_height), float(tan_fovx), float(tan_fovy),
                _ptr(means2D), _ptr(depths), _ptr(radii), _ptr(cov3D), _ptr(conic_opacity), _stream(), info=dict(P=P))
            if debug:
                _check_device(dev)
    return 0, means2D, depths, radii, cov3D, conic_opacity, rgb, clamped


def preprocess_gaussians_backward(radii, cov3D, clamped, means3D, scales, rotations, sh, scale_modifier, viewmatrix,
                                  projmatrix, tan_fovx, tan_fovy, image_height, image_width, degree, campos,
                                  dL_dmeans2D, dL_dconic_opacity, dL_dcolors, R, debug, args):
    means3D = _cuda_f32(means3D, "means3D")
    P, dev = means3D.shape[0], means3D.device
    dL_dmeans3D = torch.empty(P, 3, dtype=torch.float32, device=dev)
    dL_dscales = torch.empty(P, 3, dtype=torch.float32, device=dev)
    dL_drotations = torch.empty(P, 4, dtype=torch.float32, device=dev)
    dL_dopacity = torch.empty(P, 1, dtype=torch.float32, device=dev)
    dL_dsh = torch.zeros(P, 3, dtype=torch.float32, device=dev)
    if P:
        dm2 = _cuda_f32(dL_dmeans2D, "dL_dmeans2D")
        if dm2.shape[1] == 3:          # the reference pads the cotangent to (P,3); only x,y are used
            dm2 = dm2[:, :2].contiguous()
        with torch.cuda.device(dev):
            _call("cgx_preprocess_bwd", _lib.lib().cgx_preprocess_bwd, 
                P, _ptr(means3D), _ptr(_cuda_f32(scales, "scales")), float(scale_modifier),
                _ptr(_cuda_f32(rotations, "rotations")), _ptr(_cuda_any(radii, "radii")),
                _ptr(_cuda_f32(viewmatrix, "viewmatrix")), _ptr(_cuda_f32(projmatrix, "projmatrix")),
                int(image_width), int(image_height), float(tan_fovx), float(tan_fovy),
                _ptr(dm2), _ptr(_cuda_f32(dL_dconic_opacity, "dL_dconic_opacity")),
                _ptr(dL_dmeans3D), _ptr(dL_dscales), _ptr(dL_drotations), _ptr(dL_dopacity), _stream(), info=dict(P=P))
            if debug:
                _check_device(dev)
    return dL_dmeans3D, dL_dscales, dL_drotations, dL_dsh, dL_dopacity


def get_distribution_strategy(image_height, image_width, means2D, radii, debug, args):
    raise RuntimeError("getDistributionStrategy is deprecated.")


class _EventMs:
    """Elapsed milliseconds between two recorded CUDA events, resolved on first numeric use, so the operator
    itself never blocks the host (the reference synchronises on its timer events inside the op)."""

    def __init__(self, pairs):
        self._pairs, self._val = pairs, None

    def _get(self):
        if self._val is None:
            v = 0.0
            for a, b in self._pairs:
                b.synchronize()
                v += a.elapsed_time(b)
            self._val, self._pairs = v, None
        return self._val

    def __float__(self):
        return self._get()

    def __add__(self, o):
        return self._get() + float(o)

    __radd__ = __add__

    def __mul__(self, o):
        return self._get() * float(o)

    __rmul__ = __mul__

    def __sub__(self, o):
        return self._get() - float(o)

    def __rsub__(self, o):
        return float(o) - self._get()

    def __truediv__(self, o):
        return self._get() / float(o)

    def __repr__(self):
        return f"{self._get():.6f}"


def _stats(args):
    if isinstance(args, dict):
        return args.get("stats_collector")
    return None


def _check_device(dev):
    st = C.c_int(0)
    check(_lib.lib().cgx_device_status(C.byref(st), _stream()), "cgx_device_status")
    if st.value != 0:
        raise _lib.CgxError(st.value, "device kernel")


# ---- pair-count prefetch -------------------------------------------------------------------------------------
# render_gaussians needs the number of (tile, Gaussian) pairs on the host to size its key buffers: one host
# synchronisation per call, as in the reference (RAST/cuda_rasterizer/rasterizer_impl.cu:648-660).  A caller that
# renders several cameras in a row can start the counting stage of ALL of them first (prefetch_num_rendered), so
# that the first read-back covers every camera and the remaining launches queue back to back with no bubbles.
# render_gaussians picks a prefetched count up by the identity of its inputs; nothing changes when none exists.
_PREFETCH = {}
_PREFETCH_SLOTS = 256
_prefetch_pinned = None
_prefetch_next = 0


def _prefetch_key(means2D, radii, local, H, W):
    # the version counters make a count taken before an in-place update of its inputs unfindable
    return (means2D.data_ptr(), radii.data_ptr(), local.data_ptr(), means2D.shape[0], H, W, means2D.device.index,
            means2D._version, radii._version, local._version)


def _low_bits(dmin, dmax):
    """Varying low bits of the depth words of the sort keys, from the smallest and largest depth bit pattern."""
    dmin, dmax = dmin & 0xFFFFFFFF, dmax & 0xFFFFFFFF
    if dmin > dmax:
        return 32                      # no pairs
    return max(1, (dmin ^ dmax).bit_length())


def prefetch_num_rendered(image_height, image_width, means2D, radii, compute_locally, depths=None):
    """Launch the tile-count + prefix-sum stage of a coming render_gaussians call with these same tensors and copy
    the pair count (and, when `depths` is given, the depth range that lets the sort skip a pass) to pinned host
    memory without waiting for it.  Not part of the reference's module."""
    global _prefetch_pinned, _prefetch_next
    l = _lib.lib()
    means2D = _cuda_f32(means2D, "means2D")
    radii = _cuda_any(radii, "radii")
    local = _cuda_any(compute_locally, "compute_locally")
    P, dev = means2D.shape[0], means2D.device
    H, W = int(image_height), int(image_width)
    if P == 0 or radii.dtype != torch.int32:
        return
    if _prefetch_pinned is None:
        _prefetch_pinned = torch.zeros(_PREFETCH_SLOTS, 3, dtype=torch.int32).pin_memory()
    if len(_PREFETCH) >= _PREFETCH_SLOTS // 2:
        _PREFETCH.clear()                       # counts nobody picked up
    slot = _prefetch_next
    _prefetch_next = (_prefetch_next + 1) % _PREFETCH_SLOTS
    with torch.cuda.device(dev):
        glay = geometry_layout(P)
        geomBuffer = torch.empty(glay.total(), dtype=torch.uint8, device=dev)
        g = glay.views(geomBuffer)
        _count_scan(l, P, W, H, radii, means2D, None if depths is None else _cuda_f32(depths, "depths"), local, g,
                    _stream())
        # [1:3] only meaningful with depths; a kernel carries the words so they do not wait behind bulk read-backs
        _lib.check(l.cgx_post_words(_ptr(g["num_rendered"]), C.c_void_p(_prefetch_pinned[slot].data_ptr()), 3,
                                    _stream()), "cgx_post_words")
        ev = torch.cuda.Event()
        ev.record()
    # the tensors are kept alive with the entry, so their addresses cannot be reused while it exists
    _PREFETCH[_prefetch_key(means2D, radii, local, H, W)] = (geomBuffer, slot, ev, (means2D, radii, local),
                                                             depths is not None)


def _count_scan(l, P, W, H, radii, means2D, depths, local, g, st):
    """Tile counting + prefix sum; with depths also their range (num_rendered[1:3])."""
    if depths is None:
        _call("cgx_bin_count_scan", l.cgx_bin_count_scan, P, W, H, _ptr(radii), _ptr(means2D), _ptr(local),
              _ptr(g["tiles_touched"]), _ptr(g["num_rendered"]), _ptr(g["scanning_space"]),
              g["scanning_space"].numel(), st, info=dict(P=P))
    else:
        _call("cgx_bin_count_scan", l.cgx_bin_count_scan_depths, P, W, H, _ptr(radii), _ptr(means2D), _ptr(depths),
              _ptr(local), _ptr(g["tiles_touched"]), _ptr(g["num_rendered"]), _ptr(g["scanning_space"]),
              g["scanning_space"].numel(), st, info=dict(P=P))


def render_gaussians(background, image_height, image_width, means2D, depths, radii, conic_opacity, rgb,
                     compute_locally, viewmatrix, campos, tan_fovx, tan_fovy, all_map, render_geo, debug, args):
    l = _lib.lib()
    means2D = _cuda_f32(means2D, "means2D")
    P, dev = means2D.shape[0], means2D.device
    H, W = int(image_height), int(image_width)
    TX, TY = (W + BLOCK_X - 1) // BLOCK_X, (H + BLOCK_Y - 1) // BLOCK_Y
    T = TX * TY
    f32 = dict(dtype=torch.float32, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    n_render = torch.empty(T, **i32)
    n_consider = torch.empty(T, **i32)
    n_contrib = torch.empty(T, **i32)
    empty_u8 = torch.empty(0, dtype=torch.uint8, device=dev)
    if P == 0:
        return (0, torch.zeros(NUM_CHANNELS, H, W, **f32), n_render.zero_(), n_consider.zero_(), n_contrib.zero_(),
                torch.zeros(0, **i32), torch.zeros(NUM_ALL_MAP, H, W, **f32), torch.zeros(1, H, W, **f32),
                empty_u8, empty_u8.clone(), empty_u8.clone())

    out_color = torch.empty(NUM_CHANNELS, H, W, **f32)
    out_observe = torch.empty(P, **i32)
    out_all_map = torch.empty(NUM_ALL_MAP, H, W, **f32)
    out_plane_depth = torch.empty(1, H, W, **f32)
    depths = _cuda_f32(depths, "depths")
    radii = _cuda_any(radii, "radii").to(torch.int32)
    conic_opacity = _cuda_f32(conic_opacity, "conic_opacity")
    rgb = _cuda_f32(rgb, "rgb")
    all_map = _cuda_f32(all_map, "all_map")
    local = _cuda_any(compute_locally, "compute_locally")
    if local.dtype != torch.bool or local.numel() != T:
        raise RuntimeError("compute_locally must be a bool tensor with one entry per tile")
    if means2D.shape[1] != 2 or conic_opacity.shape != (P, 4) or rgb.shape != (P, 3) or all_map.shape != (P, 5) \
            or depths.numel() != P or radii.numel() != P:
        raise RuntimeError("render_gaussians: per-Gaussian tensors must be (P,2) (P,4) (P,3) (P,5) (P) (P)")
    bg = _cuda_f32(background, "background")
    stats = _stats(args)

    with torch.cuda.device(dev):
        st = _stream()
        glay = geometry_layout(P)
        ilay = image_layout(W * H, T)
        imgBuffer = torch.empty(ilay.total(), dtype=torch.uint8, device=dev)
        im = ilay.views(imgBuffer)
        pre = _PREFETCH.pop(_prefetch_key(means2D, radii, local, H, W), None) if _PREFETCH else None
        if pre is not None:
            geomBuffer, slot, ev, _, has_range = pre
            g = glay.views(geomBuffer)
            ev.synchronize()
            R, dmin, dmax = _prefetch_pinned[slot].tolist()
            if not has_range:
                dmin, dmax = -1, 0
        else:
            geomBuffer = torch.empty(glay.total(), dtype=torch.uint8, device=dev)
            g = glay.views(geomBuffer)
            _count_scan(l, P, W, H, radii, means2D, depths, local, g, st)
            # the key/value buffers are sized from the pair count: one host read, as in the reference
            R, dmin, dmax = g["num_rendered"][0:3].tolist()

        blay = binning_layout(R)
        binningBuffer = torch.empty(blay.total(), dtype=torch.uint8, device=dev)
        b = blay.views(binningBuffer)
        if stats is not None:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev1 = torch.cuda.Event(enable_timing=True)
            ev0.record()
        # the sort ping-pongs between the two key/value arrays: the pairs are emitted into whichever array makes
        # the last pass land in point_list_keys / point_list (no copy, whatever the number of passes)
        bit = int(l.cgx_higher_msb(T))
        # depths of one view share their leading bits: the sort squeezes them out of its digits
        low_bits = _low_bits(dmin, dmax)
        first = ("point_list_keys", "point_list") if l.cgx_sort_passes(low_bits + bit) % 2 == 0 else \
            ("point_list_keys_unsorted", "point_list_unsorted")
        other = ("point_list_keys_unsorted", "point_list_unsorted") if first[0] == "point_list_keys" else \
            ("point_list_keys", "point_list")
        _call("cgx_emit_keys", l.cgx_emit_keys, P, W, H, _ptr(radii), _ptr(means2D), _ptr(depths), _ptr(g["tiles_touched"]),
                              _ptr(local), _ptr(g["point_offsets"]), _ptr(b[first[0]]), _ptr(b[first[1]]), R,
                              _ptr(g["scanning_space"]), st, info=dict(P=P, R=R))
        _call("cgx_sort_pairs", l.cgx_sort_pairs_pingpong, R, 32 + bit, low_bits, _ptr(b[first[0]]),
                               _ptr(b[first[1]]), _ptr(b[other[0]]), _ptr(b[other[1]]), _ptr(b["list_sorting_space"]),
                               b["list_sorting_space"].numel(), 0, st, info=dict(R=R, bits=low_bits + bit))
        _call("cgx_tile_ranges", l.cgx_tile_ranges, R, T, _ptr(b["point_list_keys"]), _ptr(im["ranges"]), st, info=dict(R=R, T=T))
        _call("cgx_render_fwd", l.cgx_render_fwd, P, W, H, float(tan_fovx), float(tan_fovy), _ptr(im["ranges"]), _ptr(b["point_list"]),
                               _ptr(radii), _ptr(means2D), _ptr(rgb), _ptr(all_map), _ptr(conic_opacity), _ptr(local), _ptr(bg),
                               int(bool(render_geo)), _ptr(g["records"]), _ptr(im["accum_alpha"]),
                               _ptr(im["n_contrib"]), _ptr(im["n_contrib2loss"]), _ptr(out_color), _ptr(out_observe),
                               _ptr(out_all_map), _ptr(out_plane_depth), _ptr(n_render), _ptr(n_consider),
                               _ptr(n_contrib), st,
                               info=dict(P=P, R=R, HW=H * W, local=local, n_consider=n_consider, n_contrib=n_contrib))
        if stats is not None:
            ev1.record()
            stats["forward_render_time"] = _EventMs([(ev0, ev1)])
        _density_copy(geomBuffer, g["records"], P)
        if debug:
            _check_device(dev)
    return (R, out_color, n_render, n_consider, n_contrib, out_observe, out_all_map, out_plane_depth,
            geomBuffer, binningBuffer, imgBuffer)


# ---- density hand-over --------------------------------------------------------------------------------------
# The forward pass measures how densely the splats cover the pixel blocks they touch and leaves the counters behind
# its records; the backward pass picks its walk from them.  It can do so on the device (both kernels queued, one
# returns at once).  Cheaper: the counters are copied to pinned memory right behind the forward pass, and if they
# have arrived by the time the backward pass is queued (they have whenever something else ran in between) the
# choice is made here and one kernel is launched.  The copy is never waited for.
_DENSITY = {}
_density_pinned = None
_density_next = 0
_DENSITY_SLOTS = 256


def _density_copy(geomBuffer, records, P):
    global _density_pinned, _density_next
    n = _lib.lib().cgx_render_density_words()
    if _density_pinned is None:
        _density_pinned = torch.zeros(_DENSITY_SLOTS, n, dtype=torch.int64).pin_memory()
    if len(_DENSITY) >= _DENSITY_SLOTS // 2:
        _DENSITY.clear()                        # forward passes whose backward never came
    slot = _density_next
    _density_next = (_density_next + 1) % _DENSITY_SLOTS
    _lib.check(_lib.lib().cgx_post_words(C.c_void_p(records.data_ptr() + P * 64),
                                         C.c_void_p(_density_pinned[slot].data_ptr()), 2 * n, _stream()),
               "cgx_post_words")
    ev = torch.cuda.Event()
    ev.record()
    _DENSITY[geomBuffer.data_ptr()] = (slot, ev)


def _density_walk(geomBuffer):
    """0: let the device decide; 1: per-pixel lists; 2: every pixel looks at every visit."""
    hit = _DENSITY.pop(geomBuffer.data_ptr(), None)
    if hit is None or not hit[1].query():
        return 0
    c = _density_pinned[hit[0]]
    pixels, visits = int(c[0::2].sum()), int(c[1::2].sum())
    return 2 if pixels > _lib.lib().cgx_render_dense_threshold() * visits else 1


def render_gaussians_backward(background, tan_fovx, tan_fovy, all_map_pixels, all_maps, R, geomBuffer, binningBuffer,
                              imageBuffer, compute_locally, dL_dout_color, dL_dout_all_map, dL_dout_plane_depth,
                              means2D, conic_opacity, rgb, render_geo, debug, args):
    dL_dmeans2D, dL_dmeans2D_abs, dL_dconic_opacity, dL_dcolors, dL_dall_map = render_gaussians_backward_2d(
        background, tan_fovx, tan_fovy, all_map_pixels, all_maps, R, geomBuffer, binningBuffer, imageBuffer,
        compute_locally, dL_dout_color, dL_dout_all_map, dL_dout_plane_depth, means2D, conic_opacity, rgb, render_geo,
        debug, args)
    # the reference returns dL_dmeans2D as (P,3) with a zero third column and slices it in Python
    dL_dmeans2D_3 = torch.zeros(means2D.shape[0], 3, dtype=torch.float32, device=means2D.device)
    dL_dmeans2D_3[:, :2] = dL_dmeans2D
    return dL_dmeans2D_3, dL_dmeans2D_abs, dL_dconic_opacity, dL_dcolors, dL_dall_map


def render_gaussians_backward_2d(background, tan_fovx, tan_fovy, all_map_pixels, all_maps, R, geomBuffer,
                                 binningBuffer, imageBuffer, compute_locally, dL_dout_color, dL_dout_all_map,
                                 dL_dout_plane_depth, means2D, conic_opacity, rgb, render_geo, debug, args):
    """render_gaussians_backward with dL_dmeans2D as the (P,2) tensor the kernel writes (not an entry point of the
    reference's module: its autograd wrapper pads to (P,3) in C++ and slices back in Python; this package's wrapper
    skips the round trip)."""
    l = _lib.lib()
    P, dev = means2D.shape[0], means2D.device
    H, W = dL_dout_color.shape[1], dL_dout_color.shape[2]
    TX, TY = (W + BLOCK_X - 1) // BLOCK_X, (H + BLOCK_Y - 1) // BLOCK_Y
    f32 = dict(dtype=torch.float32, device=dev)
    dL_dmeans2D = torch.empty(P, 2, **f32)
    dL_dmeans2D_abs = torch.empty(P, 3, **f32)
    dL_dconic_opacity = torch.empty(P, 4, **f32)
    dL_dcolors = torch.empty(P, NUM_CHANNELS, **f32)
    dL_dall_map = torch.empty(P, NUM_ALL_MAP, **f32)
    if P:
        g = geometry_layout(P).views(geomBuffer)
        b = binning_layout(R).views(binningBuffer)
        im = image_layout(W * H, TX * TY).views(imageBuffer)
        stats = _stats(args)
        local = _cuda_any(compute_locally, "compute_locally")
        with torch.cuda.device(dev):
            st = _stream()
            if stats is not None:
                ev0 = torch.cuda.Event(enable_timing=True)
                ev1 = torch.cuda.Event(enable_timing=True)
                ev0.record()
            _call("cgx_render_bwd", l.cgx_render_bwd, P, W, H, float(tan_fovx), float(tan_fovy), _ptr(im["ranges"]), _ptr(b["point_list"]),
                                   _ptr(_cuda_f32(background, "background")), _ptr(g["records"]),
                                   _ptr(_cuda_f32(all_map_pixels, "all_map_pixels")), _ptr(im["accum_alpha"]),
                                   _ptr(im["n_contrib"]), _ptr(local),
                                   _ptr(_cuda_f32(dL_dout_color, "dL_dout_color")),
                                   _ptr(_cuda_f32(dL_dout_all_map, "dL_dout_all_map")),
                                   _ptr(_cuda_f32(dL_dout_plane_depth, "dL_dout_plane_depth")),
                                   int(bool(render_geo)), _ptr(dL_dmeans2D), _ptr(dL_dmeans2D_abs),
                                   _ptr(dL_dconic_opacity), _ptr(dL_dcolors), _ptr(dL_dall_map),
                                   _density_walk(geomBuffer), st, info=dict(P=P, R=R, HW=H * W, local=local))
            if stats is not None:
                ev1.record()
                stats["backward_render_time"] = _EventMs([(ev0, ev1)])
            if debug:
                _check_device(dev)
    return dL_dmeans2D, dL_dmeans2D_abs, dL_dconic_opacity, dL_dcolors, dL_dall_map


def get_local2j_ids_bool(image_height, image_width, mp_rank, mp_world_size, means2D, radii, dist_global_strategy,
                         args):
    means2D = _cuda_f32(means2D, "means2D")
    P, dev = means2D.shape[0], means2D.device
    avoid = bool(args["avoid_pixel_all2all"])
    mask = torch.empty(P, mp_world_size, dtype=torch.bool, device=dev)
    if P:
        with torch.cuda.device(dev):
            _call("cgx_local2j_mask", _lib.lib().cgx_local2j_mask, P, int(image_height), int(image_width), int(mp_world_size),
                                              _ptr(means2D), _ptr(_cuda_any(radii, "radii")),
                                              _ptr(_cuda_any(dist_global_strategy, "dist_global_strategy")
                                                   .to(torch.int32)), int(avoid),
                                              _ptr(mask), _stream())
    return mask


def get_local2j_ids_bool_adjust_mode6(image_height, image_width, mp_rank, mp_world_size, means2D, radii, rectangles,
                                      args):
    """Rectangle variant of the legacy grid strategy (RAST/rasterize_points.cu:527-603).  Off the hot path
    (its caller needs a process group the reference never creates); kept as tensor code for API completeness."""
    avoid = bool(args["avoid_pixel_all2all"])
    TX = (image_width + BLOCK_X - 1) // BLOCK_X
    TY = (image_height + BLOCK_Y - 1) // BLOCK_Y
    r = radii.to(torch.float32)
    px, py = means2D[:, 0], means2D[:, 1]

    def clamp(v, hi):
        return v.to(torch.int32).clamp(min=0).clamp(max=hi)      # C-style truncation toward zero, then clamp

    x0, y0 = clamp((px - r) / BLOCK_X, TX), clamp((py - r) / BLOCK_Y, TY)
    x1, y1 = clamp((px + r + BLOCK_X - 1) / BLOCK_X, TX), clamp((py + r + BLOCK_Y - 1) / BLOCK_Y, TY)
    rect = rectangles.to(torch.int32).clone()
    if avoid:
        rect[:, 0] = torch.where(rect[:, 0] > 0, rect[:, 0] - 1, rect[:, 0])
        rect[:, 2] = torch.where(rect[:, 2] > 0, rect[:, 2] - 1, rect[:, 2])
        rect[:, 1] += 1
        rect[:, 3] += 1
    miss = ((y1[:, None] <= rect[None, :, 0]) | (rect[None, :, 1] <= y0[:, None]) |
            (x1[:, None] <= rect[None, :, 2]) | (rect[None, :, 3] <= x0[:, None]))
    return ~miss


# Image-tile utilities of the reference's retired pixel-exchange loss modes (RAST/rasterize_points.cu:612-856).
# Off the hot path; provided as tensor code so callers that import them keep working.
def get_touched_locally(compute_locally, image_height, image_width, extension_distance):
    m = compute_locally.to(torch.float32)[None, None]
    return torch.nn.functional.max_pool2d(m, 3, stride=1, padding=1)[0, 0] > 0


def load_image_tiles_by_pos(local_image_rect, all_tiles_pos, image_height, image_width, min_pixel_y, min_pixel_x,
                            local_image_rect_height, local_image_rect_width):
    N = all_tiles_pos.shape[0]
    dev = local_image_rect.device
    ys = all_tiles_pos[:, 0, None] * BLOCK_Y + torch.arange(BLOCK_Y, device=dev)[None]      # (N, BY)
    xs = all_tiles_pos[:, 1, None] * BLOCK_X + torch.arange(BLOCK_X, device=dev)[None]      # (N, BX)
    valid = (ys < image_height)[:, :, None] & (xs < image_width)[:, None, :]
    ly = (ys - min_pixel_y).clamp(0, local_image_rect_height - 1)
    lx = (xs - min_pixel_x).clamp(0, local_image_rect_width - 1)
    tiles = local_image_rect[:, ly[:, :, None], lx[:, None, :]]                              # (3, N, BY, BX)
    tiles = torch.where(valid[None], tiles, torch.zeros((), device=dev, dtype=tiles.dtype))
    return tiles.permute(1, 0, 2, 3).contiguous() if N else tiles.new_zeros(0, 3, BLOCK_Y, BLOCK_X)


def set_image_tiles_by_pos(all_tiles_pos, image_tiles, image_height, image_width, min_pixel_y, min_pixel_x,
                           local_image_rect_height, local_image_rect_width):
    dev = image_tiles.device
    out = torch.zeros(3, local_image_rect_height, local_image_rect_width, dtype=image_tiles.dtype, device=dev)
    if all_tiles_pos.shape[0] == 0:
        return out
    ys = all_tiles_pos[:, 0, None] * BLOCK_Y + torch.arange(BLOCK_Y, device=dev)[None]
    xs = all_tiles_pos[:, 1, None] * BLOCK_X + torch.arange(BLOCK_X, device=dev)[None]
    valid = (ys < image_height)[:, :, None] & (xs < image_width)[:, None, :]
    ly = (ys - min_pixel_y)[:, :, None].expand(-1, -1, BLOCK_X)[valid]
    lx = (xs - min_pixel_x)[:, None, :].expand(-1, BLOCK_Y, -1)[valid]
    out[:, ly, lx] = image_tiles.permute(1, 0, 2, 3)[:, valid]
    return out


def get_pixels_compute_locally_and_in_rect(compute_locally, image_height, image_width, min_pixel_y, max_pixel_y,
                                           min_pixel_x, max_pixel_x):
    dev = compute_locally.device
    ys = torch.arange(min_pixel_y, max_pixel_y, device=dev) // BLOCK_Y
    xs = torch.arange(min_pixel_x, max_pixel_x, device=dev) // BLOCK_X
    return compute_locally[ys[:, None], xs[None, :]]


def rasterize_aussians_filter(means3D, scales, rotations, scale_modifier, cov3D_precomp, viewmatrix, projmatrix,
                              tan_fovx, tan_fovy, image_height, image_width, prefiltered, debug):
    if means3D.ndim != 2 or means3D.shape[1] != 3:
        raise RuntimeError("means3D must have dimensions (num_points, 3)")
    means3D = _cuda_f32(means3D, "means3D")
    P, dev = means3D.shape[0], means3D.device
    radii = torch.empty(P, dtype=torch.int32, device=dev)
    if P and cov3D_precomp is not None and cov3D_precomp.numel():
        cov = _cuda_f32(cov3D_precomp, "cov3D_precomp")
        if cov.numel() != 6 * P:
            raise RuntimeError("cov3D_precomp must hold six floats per Gaussian")
        with torch.cuda.device(dev):
            _call("cgx_filter_preprocess", _lib.lib().cgx_filter_preprocess_cov3d, P, _ptr(means3D), _ptr(cov),
                  _ptr(_cuda_f32(viewmatrix, "viewmatrix")), _ptr(_cuda_f32(projmatrix, "projmatrix")), int(image_width),
                  int(image_height), float(tan_fovx), float(tan_fovy), _ptr(radii), _stream())
    elif P:
        if scales is None or scales.numel() == 0 or rotations is None or rotations.numel() == 0:
            raise RuntimeError("visible_filter needs scales and rotations, or precomputed covariances")
        with torch.cuda.device(dev):
            _call("cgx_filter_preprocess", _lib.lib().cgx_filter_preprocess, 
                P, _ptr(means3D), _ptr(_cuda_f32(scales, "scales")), float(scale_modifier),
                _ptr(_cuda_f32(rotations, "rotations")), _ptr(_cuda_f32(viewmatrix, "viewmatrix")),
                _ptr(_cuda_f32(projmatrix, "projmatrix")), int(image_width), int(image_height), float(tan_fovx),
                float(tan_fovy), _ptr(radii), _stream())
    return radii
