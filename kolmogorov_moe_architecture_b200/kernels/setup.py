"""Build front end under the reference's path (``python moe_arch/kernels/setup.py build_ext --inplace`` there;
reference: moe_arch/kernels/setup.py).  The reference picks ``-gencode`` flags from the GPU it finds; this library is
written for one architecture, so the flags are fixed and the build needs no GPU (nvcc cross-compiles):

    python -m kolmogorov_moe_architecture_b200.kernels.setup [build_ext] [--inplace] [--force]

which is the same as ``python build_ext.py`` at the repository root.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from typing import List, Optional, Tuple

ARCH = "sm_100a"


def get_cuda_version() -> Optional[Tuple[int, int]]:
    """(major, minor) of the nvcc on the path (or under ``/usr/local/cuda``), None without one."""
    for nvcc in (os.environ.get("NVCC"), "nvcc", "/usr/local/cuda/bin/nvcc"):
        if not nvcc:
            continue
        try:
            out = subprocess.run([nvcc, "--version"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True).stdout
        except OSError:
            continue
        m = re.search(r"release (\d+)\.(\d+)", out)
        if m:
            return int(m.group(1)), int(m.group(2))
    return None


def get_gpu_arch() -> Optional[Tuple[int, int]]:
    """Compute capability of GPU 0, None without a GPU."""
    try:
        import torch
        if torch.cuda.is_available():
            return tuple(torch.cuda.get_device_capability(0))
    except Exception:
        pass
    return None


def get_cuda_arch_flags() -> List[str]:
    """The one architecture this library is written for: tcgen05 / TMEM / TMA instructions exist in the
    architecture-specific ``sm_100a`` target only."""
    ver = get_cuda_version()
    if ver is not None and ver < (12, 8):
        raise RuntimeError(f"CUDA {ver[0]}.{ver[1]} cannot target {ARCH}; 12.8 or newer is needed")
    return ["-gencode", "arch=compute_100a,code=sm_100a"]


def main(argv=None) -> str:
    argv = list(sys.argv[1:] if argv is None else argv)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    import build_ext
    return build_ext.build(force="--force" in argv)


if __name__ == "__main__":
    main()
