"""The C-ABI library loads and exports every symbol the public header declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols(headers=("cgx_raster.h", "cgx_raster_testing.h")):
    """Entry points of the drop-in boundary (cgx_raster.h) and of the test-only switches (cgx_raster_testing.h)."""
    names = set()
    for h in headers:
        text = (ROOT / "include" / h).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(cgx_\w+)\s*\(", text))
    return sorted(names)


def test_header_symbols_are_exported():
    from diff_gaussian_rasterization import _lib

    so = _lib.build()
    handle = ctypes.CDLL(str(so))
    names = declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(handle, n)]
    assert not missing, f"declared in cgx_raster.h but not exported: {missing}"


def test_binding_table_matches_header():
    from diff_gaussian_rasterization import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()
    # the public header holds no process-wide switches: those live in the test-only header
    assert not [n for n in declared_symbols(("cgx_raster.h",)) if "_set_" in n]


def test_host_only_entry_points():
    from diff_gaussian_rasterization import _lib

    l = _lib.lib()
    bx, by, od = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    assert l.cgx_block_xy(ctypes.byref(bx), ctypes.byref(by), ctypes.byref(od)) == 0
    assert (bx.value, by.value, od.value) == (16, 16, 256)
    # next-highest bit of the MSB, as used for the number of sorted key bits
    for n, want in [(1, 1), (2, 2), (144, 8), (7500, 13), (8160, 13), (8192, 14), (32400, 15), (65535, 16)]:
        assert l.cgx_higher_msb(n) == want
    assert l.cgx_strerror(22).decode().startswith("invalid argument")
    assert l.cgx_preprocess_fwd(-1, None, None, 1.0, None, None, None, None, 8, 8, 1.0, 1.0,
                                None, None, None, None, None, None) == _lib.CGX_EINVAL
    assert l.cgx_sort_workspace_bytes(1 << 20) >= (1 << 20) // 4096 * 256 * 4


def test_package_surface():
    import diff_gaussian_rasterization as d

    for name in ("GaussianRasterizationSettings", "GaussianRasterizer", "preprocess_gaussians", "render_gaussians",
                 "load_image_tiles_by_pos", "merge_image_tiles_by_pos", "_C"):
        assert hasattr(d, name)
    for name in ("mark_visible", "preprocess_gaussians", "preprocess_gaussians_backward", "get_distribution_strategy",
                 "render_gaussians", "render_gaussians_backward", "get_local2j_ids_bool",
                 "get_local2j_ids_bool_adjust_mode6", "get_touched_locally", "load_image_tiles_by_pos",
                 "set_image_tiles_by_pos", "get_pixels_compute_locally_and_in_rect", "get_block_XY",
                 "rasterize_aussians_filter"):
        assert callable(getattr(d._C, name)), name
    assert d._C.get_block_XY() == (16, 16, 256)
    assert d.GaussianRasterizationSettings._fields == (
        "image_height", "image_width", "tanfovx", "tanfovy", "bg", "scale_modifier", "viewmatrix", "projmatrix",
        "sh_degree", "campos", "prefiltered", "render_geo", "debug")


def test_cpu_tensors_are_refused():
    import pytest
    import torch
    import diff_gaussian_rasterization as d

    with pytest.raises(RuntimeError, match="CUDA"):
        d._C.mark_visible(torch.zeros(4, 3), torch.eye(4), torch.eye(4))
