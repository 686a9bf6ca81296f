"""Build the in-tree CUDA extension ``kolmogorov_moe_architecture_b200/_C.so``.

    python build_ext.py            # incremental (mtime based)
    python build_ext.py --force    # rebuild everything
    python build_ext.py --ptxas-v  # print register / shared-memory usage

Every ``csrc/*.cu`` is compiled for sm_100a only (``-gencode
arch=compute_100a,code=sm_100a -lineinfo``); kernels are torch-free so each file
takes seconds.  ``csrc/bindings.cpp`` (the only file that includes torch
headers) is compiled with the host compiler.  nvcc cross-compiles, so this runs
on a machine without a GPU.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "kolmogorov_moe_architecture_b200")
SRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
OUT = os.path.join(PKG, "_C.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-I/usr/local/cuda/include"]


def _newer(src: str, dst: str, deps) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(p) > t for p in [src, *deps])


def _run(cmd, quiet=False):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + "\n")
        raise RuntimeError(f"build step failed: {cmd[0]} ... {cmd[-1]}")
    if not quiet and r.stdout.strip():
        print(r.stdout)
    return r.stdout


def build(force: bool = False, ptxas_v: bool = False, verbose: bool = True) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(SRC, f) for f in os.listdir(SRC) if f.endswith((".h", ".cuh"))]
    cus = sorted(f for f in os.listdir(SRC) if f.endswith(".cu"))
    objs, jobs = [], []
    for f in cus:
        src, obj = os.path.join(SRC, f), os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or ptxas_v or _newer(src, obj, headers):
            cmd = [NVCC, *NVCC_FLAGS, *(["-Xptxas", "-v"] if ptxas_v else []), "-c", src, "-o", obj]
            jobs.append(cmd)
    bsrc, bobj = os.path.join(SRC, "bindings.cpp"), os.path.join(OBJ, "bindings.o")
    objs.append(bobj)
    if force or _newer(bsrc, bobj, headers):
        inc = [f"-I{p}" for p in ce.include_paths()] + ["-I/usr/local/cuda/include"]
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        jobs.append([CXX, "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                     "-DTORCH_EXTENSION_NAME=_C", *inc, "-c", bsrc, "-o", bobj])
    if jobs:
        if verbose:
            print(f"[build_ext] compiling {len(jobs)} file(s)")
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, quiet=not ptxas_v), jobs))
    if jobs or not os.path.exists(OUT):
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        # The C++ runtime must be the process-wide shared one.  A toolchain whose search path only offers
        # libstdc++.a would otherwise put a private copy of the runtime into the library; its stream / locale
        # state is then not the one libtorch initialised, and the first formatted error message (TORCH_CHECK
        # with a number in it) crashes instead of raising.  Hence: no implicit -lstdc++, the shared object by name.
        _run([CXX, "-shared", "-nostdlib++", "-o", OUT, *objs, f"-L{tlib}", "-lc10", "-ltorch_cpu", "-ltorch",
              "-lc10_cuda", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart", "-l:libstdc++.so.6", "-lm",
              f"-Wl,-rpath,{tlib}", "-Wl,-rpath,/usr/local/cuda/lib64"])
        private = _run(["nm", "-D", "--defined-only", OUT], quiet=True).count("_ZNSt6locale5_Impl")
        if private:
            raise RuntimeError(f"{OUT} contains a private copy of the C++ runtime ({private} std::locale symbols)")
        if verbose:
            print(f"[build_ext] linked {OUT}")
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true")
    a = ap.parse_args()
    build(a.force, a.ptxas_v)
