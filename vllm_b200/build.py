"""In-tree build of the native libraries (sm_100a only).

``libb200pa.so``  the C-ABI library (CUDA kernels + launchers, links cudart only)
``_C_b200.so``    the PyTorch registration shim (links libb200pa.so and torch)

Both land next to this file so they travel with the working tree.  Usage::

    python -m vllm_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libb200pa.so"
SHIM = PKG / "_C_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:4])} ...")
    if verbose and r.stdout.strip():
        print(r.stdout)


def build_lib(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "b200pa.h"]
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [NVCC, "-c", str(src), "-o", str(obj)] + NVCC_FLAGS
            if verbose:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or _newer(LIB, objs):
        _run([NVCC, "-shared", "-o", str(LIB)] + [str(o) for o in objs] +
             ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"], verbose)
    return LIB


def build_shim(force: bool = False, verbose: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    src = CSRC / "torch_shim.cpp"
    if not (force or _newer(SHIM, [src, LIB, PKG.parent / "include" / "b200pa.h"])):
        return SHIM
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}",
                                                   "-I/usr/local/cuda/include"]
    cmd = ["g++", "-shared", "-fPIC", "-O2", "-std=c++17", "-D_GLIBCXX_USE_CXX11_ABI=1",
           str(src), "-o", str(SHIM)] + inc + [
        f"-L{PKG}", "-lb200pa", f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
        "-lc10_cuda", "-L/usr/local/cuda/lib64", "-lcudart",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    _run(cmd, verbose)
    return SHIM


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_lib(force, verbose)
    build_shim(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    build_all(a.force, a.verbose)
    print(f"built {LIB.name}, {SHIM.name}")
