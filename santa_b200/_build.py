"""In-tree build of the native pieces.

* ``libsanta_b200.so`` -- the C-ABI CUDA library (``csrc/*.cu``), compiled by
  nvcc for sm_100a only.  The Flash translation unit is compiled with
  ``--use_fast_math`` and the Prop unit without, mirroring the reference's two
  extensions: the sampled row counts depend on those floating-point modes.
* ``santa_flash_batch_cuda`` / ``santa_prop_batch_cuda`` -- thin pybind11/ATen
  extension modules over that library exposing the reference's Python operator
  surface (built with torch.utils.cpp_extension, no CUDA code of their own).

Everything lands in ``santa_b200/lib`` so that the built files travel with the
source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_PKG, "csrc")
LIBDIR = os.path.join(_PKG, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB_PATH = os.path.join(LIBDIR, "libsanta_b200.so")
INCLUDE = os.path.join(os.path.dirname(_PKG), "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# translation unit -> extra flags
UNITS = {
    "flash_kernels.cu": ["--use_fast_math"],
    "prop_kernels.cu": [],
    "combine_kernels.cu": [],
    "capi.cu": [],
}


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "santa_b200.h"))
    return hs


def build_library(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdrs = _headers()
    objs = []
    procs = []
    for unit, extra in UNITS.items():
        src = os.path.join(CSRC, unit)
        if not os.path.exists(src):
            continue
        obj = os.path.join(OBJDIR, unit.replace(".cu", ".o"))
        objs.append(obj)
        if not force and _newer(obj, [src] + hdrs):
            continue
        cmd = [nvcc] + ARCH + COMMON + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((unit, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for unit, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(out)
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {unit}")
    if force or procs or not _newer(LIB_PATH, objs):
        cmd = [nvcc] + ARCH + ["-shared", "-o", LIB_PATH] + objs
        subprocess.check_call(cmd)
    return LIB_PATH


EXT_MODULES = {
    "santa_flash_batch_cuda": "torch_flash.cpp",
    "santa_prop_batch_cuda": "torch_prop.cpp",
}


def build_extensions(verbose: bool = False) -> None:
    """Build the two pybind11/ATen modules into ``santa_b200/lib``."""
    from torch.utils import cpp_extension

    for name, src in EXT_MODULES.items():
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        sofile = os.path.join(LIBDIR, name + ".so")
        if _newer(sofile, [path, LIB_PATH] + _headers()):
            continue
        build_dir = os.path.join(OBJDIR, name)
        os.makedirs(build_dir, exist_ok=True)
        cpp_extension.load(
            name=name,
            sources=[path],
            extra_cflags=["-O2", "-std=c++17"],
            extra_include_paths=[INCLUDE, os.path.join(cpp_extension.CUDA_HOME, "include")],
            extra_ldflags=[f"-L{LIBDIR}", "-lsanta_b200", "-Wl,-rpath,$ORIGIN"],
            build_directory=build_dir,
            with_cuda=True,
            is_python_module=False,
            verbose=verbose,
        )
        built = os.path.join(build_dir, name + ".so")
        os.replace(built, sofile)


def build_all(verbose: bool = False) -> None:
    build_library(verbose=verbose)
    build_extensions(verbose=verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
