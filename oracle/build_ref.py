"""Build recipe for the GPU-side checker: the reference's own CUDA rasterizer.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file
or its output.

The reference rasterizer (submodule_cityx/diff-gaussian-rasterization) is CUDA
only; it has no CPU path.  This script compiles the reference's six source
files *where they lie* in a read-only checkout (nothing is copied) with plain
``nvcc`` calls into ``oracle/_ref/cityx_ref_C.so``, a pybind11 module exposing
the reference's raw ``_C`` entry points (ext.cpp:17-34).  The GPU parity tests
call those entry points directly on identical inputs to check radii, sorted
keys, tile ranges (bit-exact) and the float outputs/gradients (tolerances).

It does not run the reference's setup.py.  Flags mirror what that build would
use (no fast-math, default -fmad, -std=c++17, --expt-relaxed-constexpr, glm on
the include path) so the arithmetic is the reference's.

Usage:  python oracle/build_ref.py [--src DIR]   (DIR defaults to
``$CGX_REFERENCE_RAST`` or the conventional checkout location).
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
MODULE = "cityx_ref_C"
# default location: a checkout of the reference next to this repository (<parent>/reference)
DEFAULT_SRC = str(HERE.parent.parent / "reference" / "submodule_cityx" / "diff-gaussian-rasterization")

SOURCES = [
    "cuda_rasterizer/rasterizer_impl.cu",
    "cuda_rasterizer/forward.cu",
    "cuda_rasterizer/backward.cu",
    "cuda_rasterizer/timers.cu",
    "rasterize_points.cu",
    "ext.cpp",
]


def reference_dir(arg: str | None = None) -> Path | None:
    cand = arg or os.environ.get("CGX_REFERENCE_RAST") or DEFAULT_SRC
    p = Path(cand)
    return p if (p / "ext.cpp").is_file() else None


def so_path() -> Path:
    return OUT / f"{MODULE}.so"


def build(src: Path, force: bool = False, verbose: bool = True) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    OUT.mkdir(exist_ok=True)
    target = so_path()
    newest_src = max((src / s).stat().st_mtime for s in SOURCES)
    if target.exists() and not force and target.stat().st_mtime > max(
        newest_src, Path(__file__).stat().st_mtime
    ):
        return target

    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    incs = ce.include_paths("cuda") + [sysconfig.get_paths()["include"], str(src / "third_party/glm")]
    common = [f"-I{i}" for i in incs] + [
        f"-DTORCH_EXTENSION_NAME={MODULE}",
        "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        "-std=c++17",
    ]
    nv_flags = [
        "-gencode=arch=compute_100,code=sm_100",
        "--expt-relaxed-constexpr",
        "-D__CUDA_NO_HALF_OPERATORS__",
        "-D__CUDA_NO_HALF_CONVERSIONS__",
        "-D__CUDA_NO_BFLOAT16_CONVERSIONS__",
        "-D__CUDA_NO_HALF2_OPERATORS__",
        "-O3",
        "--compiler-options",
        "-fPIC",
        "-w",
    ]

    def compile_one(rel: str) -> Path:
        obj = OUT / (rel.replace("/", "_") + ".o")
        cmd = [nvcc, "-c", str(src / rel), "-o", str(obj)] + common + nv_flags
        if verbose:
            print("[build_ref]", rel, flush=True)
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(6, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, SOURCES))

    libdirs = ce.library_paths("cuda")
    link = (
        [nvcc, "-shared", "-o", str(target)]
        + [str(o) for o in objs]
        + [f"-L{d}" for d in libdirs]
        + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    )
    subprocess.run(link, check=True)
    for o in objs:
        o.unlink()
    return target


def load():
    """Import the built module (torch must be imported first so its libraries resolve)."""
    import importlib.util

    import torch  # noqa: F401

    p = so_path()
    if not p.exists():
        return None
    spec = importlib.util.spec_from_file_location(MODULE, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    s = reference_dir(a.src)
    if s is None:
        print("[build_ref] reference sources not found; nothing built")
        sys.exit(0)
    print(build(s, force=a.force))
