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
    "rope_kernels.cu": [],
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


CHECKS_LIB_PATH = os.path.join(LIBDIR, "libsanta_b200_checks.so")


def build_library(verbose: bool = False, force: bool = False, checks: bool = False) -> str:
    """Compile the C-ABI library.  ``checks=True`` builds ``libsanta_b200_checks.so`` instead: the same
    sources with -DSANTA_B200_CHECKS, every data-dependent index compared with its array's extent and
    violations reported through the status word (select it with the SANTA_B200_LIB environment
    variable; see santa_b200/capi.py)."""
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdrs = _headers()
    objs = []
    procs = []
    lib_path = CHECKS_LIB_PATH if checks else LIB_PATH
    for unit, extra in UNITS.items():
        src = os.path.join(CSRC, unit)
        if not os.path.exists(src):
            continue
        if checks:
            extra = extra + ["-DSANTA_B200_CHECKS"]
        obj = os.path.join(OBJDIR, unit.replace(".cu", ".checks.o" if checks else ".o"))
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
    if force or procs or not _newer(lib_path, objs):
        cmd = [nvcc] + ARCH + ["-shared", "-o", lib_path] + objs
        subprocess.check_call(cmd)
    return lib_path


EXT_MODULES = {
    "santa_flash_batch_cuda": "torch_flash.cpp",
    "santa_prop_batch_cuda": "torch_prop.cpp",
}


def build_extensions(verbose: bool = False) -> None:
    """Build the two pybind11/ATen modules into ``santa_b200/lib`` with one g++ call each."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    cxx = os.environ.get("CXX", "g++")
    inc = [INCLUDE, sysconfig.get_paths()["include"]] + cpp_extension.include_paths("cuda")
    libdirs = cpp_extension.library_paths("cuda")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for name, src in EXT_MODULES.items():
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        sofile = os.path.join(LIBDIR, name + ".so")
        if _newer(sofile, [path, LIB_PATH, os.path.join(INCLUDE, "santa_b200.h")]):
            continue
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", path, "-o", sofile,
               f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
        cmd += [f"-I{d}" for d in inc]
        cmd += [f"-L{d}" for d in libdirs] + [f"-L{LIBDIR}"]
        cmd += ["-lsanta_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
                "-Wl,-rpath,$ORIGIN"] + [f"-Wl,-rpath,{d}" for d in libdirs if "torch" in d]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)


def build_all(verbose: bool = False) -> None:
    build_library(verbose=verbose)
    build_extensions(verbose=verbose)


if __name__ == "__main__":
    if "--checks" in sys.argv:
        print(build_library(verbose="-v" in sys.argv, checks=True))
    else:
        build_all(verbose="-v" in sys.argv)
