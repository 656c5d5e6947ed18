"""Build the in-tree CUDA extension ``sample_efficient_gpt_b200/_C.so`` for sm_100a.

``python -m sample_efficient_gpt_b200.csrc.build [--force] [--debug-bounds]``.  Every ``.cu`` file is compiled by nvcc with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` (no framework headers, seconds per file), the binding
translation units by g++ against the torch headers, and everything is linked into one shared object next to the
package so that it travels with the source tree.  Objects are rebuilt only when their sources changed.
``--debug-bounds`` builds a second module, ``_C_dbg.so``, from the same sources with ``-DSEG_DEBUG_BOUNDS``: its kernels
check every computed store index against the extent of its destination (``bounds.cuh``); ``SEGPT_DEBUG_BOUNDS=1`` makes
the package load it instead of ``_C.so``.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
OBJ = HERE / "build"
TARGET = PKG / "_C.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    mod = "_C_dbg" if debug_bounds else "_C"
    target = PKG / f"{mod}.so"
    flavour = ["-DSEG_DEBUG_BOUNDS"] if debug_bounds else []
    obj_dir = HERE / "build_dbg" if debug_bounds else OBJ
    obj_dir.mkdir(exist_ok=True)
    headers = list(HERE.glob("*.h")) + list(HERE.glob("*.cuh"))
    hdig = _digest(headers)
    cu_files = sorted(HERE.glob("*.cu"))
    cpp_files = sorted(HERE.glob("*.cpp"))
    jobs, objs = [], []
    cuda_home = Path(NVCC).resolve().parent.parent
    for src in cu_files:
        tag = _digest([src]) + hdig
        obj = obj_dir / f"{src.stem}.{tag}.o"
        objs.append(obj)
        if force or not obj.exists():
            for old in obj_dir.glob(f"{src.stem}.*.o"):
                old.unlink()
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append([NVCC, *ARCH, "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                         *flavour, *extra, "-I", str(HERE), "-c", str(src), "-o", str(obj)])
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{cuda_home}/include", f"-I{sysconfig.get_paths()['include']}", f"-I{HERE}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for src in cpp_files:
        tag = _digest([src]) + hdig + torch.__version__.replace("+", "_")
        obj = obj_dir / f"{src.stem}.{tag}.o"
        objs.append(obj)
        if force or not obj.exists():
            for old in obj_dir.glob(f"{src.stem}.*.o"):
                old.unlink()
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DTORCH_EXTENSION_NAME={mod}", *flavour,
                         "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", str(src), "-o", str(obj)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(_run, jobs):
                if verbose and out.strip():
                    print(out)
    if jobs or force or not target.exists():
        torch_lib = Path(torch.__file__).parent / "lib"
        _run(["g++", "-shared", "-o", str(target), *map(str, objs), f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
              "-ltorch_cuda", "-ltorch", "-ltorch_python", f"-L{cuda_home}/lib64", "-lcudart", f"-Wl,-rpath,{torch_lib}"])
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_bounds="--debug-bounds" in sys.argv)
    print(path)
