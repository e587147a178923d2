"""ctypes binding of libcgx_raster.so (the C ABI declared in include/cgx_raster.h).

The library is built in-tree by ``build()`` (plain nvcc, sm_100a).  There is no CPU fallback: if the
shared library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
# CGX_RASTER_LIB: load another build of the same library (A/B timing of compile-time tile sizes); never a fallback
SO = Path(os.environ["CGX_RASTER_LIB"]) if os.environ.get("CGX_RASTER_LIB") else LIBDIR / "libcgx_raster.so"
SOURCES = ["cabi.cu", "preprocess.cu", "binning.cu", "render.cu", "peer.cu", "loss.cu", "redistribute.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]

CGX_OK, CGX_EINVAL, CGX_ENOMEM, CGX_ETIMEDOUT, CGX_ECUDA = 0, 22, 12, 110, 5


def sources():
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into lib/libcgx_raster.so when out of date."""
    srcs = sources()
    deps = srcs + [CSRC / "cgx_common.cuh", ROOT.parent / "include" / "cgx_raster.h",
                   ROOT.parent / "include" / "cgx_raster_testing.h"]
    newest = max(p.stat().st_mtime for p in deps if p.exists())
    if not force and SO.exists() and SO.stat().st_mtime >= newest:
        return SO
    LIBDIR.mkdir(exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + [str(s) for s in srcs] + ["-o", str(SO)]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)
    return SO


_vp, _i, _f, _i64, _sz = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_size_t

# name -> (restype, argtypes); mirrors include/cgx_raster.h one to one
SIGNATURES = {
    "cgx_strerror": (C.c_char_p, [_i]),
    "cgx_last_cuda_error": (C.c_char_p, []),
    "cgx_version": (C.c_char_p, []),
    "cgx_block_xy": (_i, [_vp, _vp, _vp]),
    "cgx_higher_msb": (C.c_uint32, [C.c_uint32]),
    "cgx_mark_visible": (_i, [_i, _vp, _vp, _vp, _vp]),
    "cgx_preprocess_fwd": (_i, [_i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_filter_preprocess": (_i, [_i, _vp, _vp, _f, _vp, _vp, _vp, _i, _i, _f, _f, _vp, _vp]),
    "cgx_filter_preprocess_cov3d": (_i, [_i, _vp, _vp, _vp, _vp, _i, _i, _f, _f, _vp, _vp]),
    "cgx_sh_to_rgb": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_preprocess_bwd": (_i, [_i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_preprocess_fwd_batched": (_i, [_i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_preprocess_bwd_batched": (_i, [_i, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_preprocess_fwd_batched_planes": (_i, [_i, _i, _vp, _vp, _f] + [_vp] * 10),
    "cgx_preprocess_bwd_batched_planes": (_i, [_i, _i, _vp, _vp, _f] + [_vp] * 12),
    "cgx_preprocess_bwd_rows_workspace_bytes": (_sz, [_i]),
    "cgx_preprocess_bwd_rows": (_i, [_i, _i, _vp, _i, _vp, _vp, _vp, _vp, _f, _vp, _i, _vp, _vp, _vp, _sz,
                                     _vp, _vp, _vp, _vp, _vp]),
    "cgx_all_map_fwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_all_map_bwd": (_i, [_i] + [_vp] * 10),
    "cgx_strip_loss_fwd": (_i, [_i, _i, _i] + [_vp] * 8),
    "cgx_strip_loss_bwd": (_i, [_i, _i, _i] + [_vp] * 9),
    "cgx_depth_normal_fwd": (_i, [_i, _i, _f, _f, _f, _f, _vp, _vp, _vp]),
    "cgx_depth_normal_bwd": (_i, [_i, _i, _f, _f, _f, _f, _vp, _vp, _vp, _vp]),
    "cgx_local2j_mask": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp]),
    "cgx_local2j_count": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _sz, _vp]),
    "cgx_local2j_count_batched": (_i, [_i, _vp, _vp]),
    "cgx_local2j_workspace_bytes": (_sz, [_i, _i]),
    "cgx_local2j_pack": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "cgx_unpack_grad_add": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_unpack_rows": (_i, [_i] + [_vp] * 13),
    "cgx_pack_grad_rows": (_i, [_i] + [_vp] * 10),
    "cgx_local2j_pack_p2p": (_i, [_i, _i, _i, _i] + [_vp] * 9 + [_i] + [_vp] * 4 + [_sz, _vp]),
    "cgx_local2j_pack_p2p_batched": (_i, [_i, _vp, _vp, _vp]),
    "cgx_pack_grad_rows_to": (_i, [_i, _vp, _vp, _i, _i] + [_vp] * 7),
    "cgx_unpack_grad_add_cols": (_i, [_i, _vp, _vp, _i] + [_vp] * 9),
    "cgx_rows_workspace_bytes": (_sz, [_i64, _i]),
    "cgx_rows_dest_count": (_i, [_i64, _i, _vp, _vp, _vp, _sz, _vp]),
    "cgx_rows_pack": (_i, [_i64, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cgx_rows_unpack": (_i, [_i64, _vp, _i, _vp, _vp, _vp]),
    "cgx_peer_barrier": (_i, [_i, _i, _vp, C.c_uint32, _vp]),
    "cgx_peer_barrier_limited": (_i, [_i, _i, _vp, C.c_uint32, C.c_uint64, _vp]),
    "cgx_bin_workspace_bytes": (_sz, [_i]),
    "cgx_bin_count_scan": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "cgx_bin_count_scan_depths": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "cgx_emit_keys": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "cgx_sort_workspace_bytes": (_sz, [_i64]),
    "cgx_sort_pairs": (_i, [_i64, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "cgx_sort_passes": (_i, [_i]),
    "cgx_sort_pairs_pingpong": (_i, [_i64, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, C.c_uint64, _vp]),
    "cgx_sort_pairs_static_max": (_i64, []),
    "cgx_sort_pairs_static": (_i, [_i64, _i, _vp, _vp, _vp, _vp, _vp]),
    "cgx_set_sort_variant": (_i, [_i]),
    "cgx_tile_ranges": (_i, [_i64, _i, _vp, _vp, _vp]),
    "cgx_render_records_bytes": (_sz, [_i]),
    "cgx_render_fwd": (_i, [_i, _i, _i, _f, _f] + [_vp] * 9 + [_i] + [_vp] * 12),
    "cgx_launch_count": (C.c_uint64, []),
    "cgx_tile_stats": (_i, [_i, _i] + [_vp] * 8),
    "cgx_render_bwd": (_i, [_i, _i, _i, _f, _f] + [_vp] * 11 + [_i] + [_vp] * 5 + [_i, _vp]),
    "cgx_render_density_words": (_i, []),
    "cgx_render_dense_threshold": (_i, []),
    "cgx_device_status": (_i, [_vp, _vp]),
    "cgx_device_status_async": (_i, [_vp, _vp]),
    "cgx_post_words": (_i, [_vp, _vp, _i, _vp]),
    "cgx_set_render_variant": (_i, [_i]),
}

_lib = None


def lib():
    """The loaded shared library.  Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not SO.exists():
            raise ImportError(
                f"{SO} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(needs nvcc); this package has no CPU or PyTorch fallback")
        handle = C.CDLL(str(SO))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)      # AttributeError here means header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class CgxError(RuntimeError):
    def __init__(self, status: int, where: str):
        l = lib()
        msg = l.cgx_strerror(status).decode()
        if status == CGX_ECUDA:
            msg += ": " + l.cgx_last_cuda_error().decode()
        super().__init__(f"{where} failed with status {status} ({msg})")
        self.status = status


def current_stream_ptr() -> int:
    """cudaStream_t of torch's current stream on the current device, as an integer (the raw getters: the
    torch.cuda.current_stream() object costs tens of microseconds per call and this sits before every launch)."""
    import torch

    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def check(status: int, where: str):
    if status != CGX_OK:
        raise CgxError(status, where)
