"""Build the reference project's own kernels into ``oracle/_ref/`` (TEST INFRASTRUCTURE).

Two libraries are produced from sources compiled *where they lie* in the
reference checkout (nothing is copied into this repository):

``_C_ref.so``
    csrc/attention/paged_attention_v1.cu, csrc/attention/paged_attention_v2.cu and
    csrc/cache_kernels.cu of the reference, compiled unmodified for sm_100a and
    registered by ``ref_cuda_binding.cpp`` as ``torch.ops._C_ref.*`` /
    ``torch.ops._C_ref_cache_ops.*``.  GPU parity oracle.

``_C_ref_cpu.so``
    csrc/cpu/cpu_attn.cpp + csrc/cpu/scratchpad_manager.cpp (the reference's CPU
    decode attention), registered by ``ref_cpu_binding.cpp`` as
    ``torch.ops._C_ref_cpu.*``.  Pins the CPU oracle and is the timed CPU baseline.

The reference's own build system (cmake + downloads) is not run.  Usage::

    python oracle/build_ref.py [--reference /path/to/reference] [--only cuda|cpu]

The script is a no-op (exit 0) when the reference checkout is absent, so the
prebuilt libraries that travelled with the working tree keep being used.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    return inc, lib


def _run(cmd: list[str], log: Path) -> None:
    t0 = time.time()
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n")
        f.flush()
        rc = subprocess.call(cmd, stdout=f, stderr=subprocess.STDOUT)
    if rc != 0:
        sys.stderr.write(f"FAILED ({rc}): see {log}\n")
        raise SystemExit(rc)
    print(f"  ok {time.time() - t0:6.1f}s  {log.name}", flush=True)


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources if s.exists())


def build_cuda(ref: Path, force: bool) -> None:
    inc, lib = _torch_paths()
    csrc = ref / "csrc"
    cu = [
        csrc / "attention" / "paged_attention_v1.cu",
        csrc / "attention" / "paged_attention_v2.cu",
        csrc / "cache_kernels.cu",
    ]
    binding = HERE / "ref_cuda_binding.cpp"
    target = OUT / "_C_ref.so"
    if not force and not _stale(target, cu + [binding]):
        print("oracle/_ref/_C_ref.so is up to date")
        return
    pyinc = sysconfig.get_paths()["include"]
    common = ["-std=c++17", "-O2", "-DENABLE_FP8", "-D_GLIBCXX_USE_CXX11_ABI=1",
              f"-I{csrc}", f"-I{pyinc}"] + [f"-I{p}" for p in inc]
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    jobs = []
    for src in cu:
        obj = OUT / (src.stem + ".o")
        objs.append(obj)
        jobs.append(([nvcc, "-c", str(src), "-o", str(obj),
                      "-gencode", "arch=compute_100a,code=sm_100a",
                      "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"] + common,
                     OUT / (src.stem + ".log")))
    bobj = OUT / "ref_cuda_binding.o"
    objs.append(bobj)
    jobs.append((["g++", "-c", str(binding), "-o", str(bobj), "-fPIC"] + common,
                 OUT / "ref_cuda_binding.log"))
    print("building _C_ref.so (reference CUDA kernels, sm_100a; several minutes)", flush=True)
    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(lambda j: _run(*j), jobs))
    _run(["g++", "-shared", "-o", str(target)] + [str(o) for o in objs] +
         [f"-L{lib}", "-L/usr/local/cuda/lib64", "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
          "-lc10", "-lc10_cuda", "-lcudart", f"-Wl,-rpath,{lib}"],
         OUT / "link_cuda.log")


def build_cpu(ref: Path, force: bool) -> None:
    inc, lib = _torch_paths()
    csrc = ref / "csrc"
    srcs = [csrc / "cpu" / "cpu_attn.cpp", csrc / "cpu" / "scratchpad_manager.cpp",
            HERE / "ref_cpu_binding.cpp"]
    target = OUT / "_C_ref_cpu.so"
    if not force and not _stale(target, srcs):
        print("oracle/_ref/_C_ref_cpu.so is up to date")
        return
    print("building _C_ref_cpu.so (reference CPU attention)", flush=True)
    cmd = ["g++", "-shared", "-fPIC", "-O2", "-std=c++17", "-fopenmp",
           "-mavx512f", "-mavx512vl", "-mavx512bw", "-mavx512dq", "-mf16c",
           "-D_GLIBCXX_USE_CXX11_ABI=1", f"-I{csrc}", f"-I{csrc / 'cpu'}"]
    cmd += [f"-I{p}" for p in inc if "cuda" not in p]
    cmd += [str(s) for s in srcs]
    cmd += ["-o", str(target), f"-L{lib}", "-ltorch", "-ltorch_cpu", "-lc10",
            f"-Wl,-rpath,{lib}"]
    _run(cmd, OUT / "build_cpu.log")


def main() -> int:
    ap = argparse.ArgumentParser()
    # default: $VLLM_REFERENCE_DIR, else a checkout named "reference" beside this repository
    ap.add_argument("--reference", default=os.environ.get("VLLM_REFERENCE_DIR",
                                                          str(HERE.parent.parent / "reference")))
    ap.add_argument("--only", choices=["cuda", "cpu"])
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    ref = Path(a.reference)
    if not (ref / "csrc").is_dir():
        print(f"reference checkout not found at {ref}: keeping prebuilt oracle/_ref")
        return 0
    OUT.mkdir(exist_ok=True)
    if a.only in (None, "cpu"):
        build_cpu(ref, a.force)
    if a.only in (None, "cuda"):
        build_cuda(ref, a.force)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
