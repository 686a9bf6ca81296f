#!/bin/bash
# Build the CUDA kernels of kolmogorov_moe_architecture_b200 (in-tree shared library, sm_100a only).
#
#   ./build_kernels.sh [--force]
#
# Needs nvcc (CUDA 12.8 or newer: the kernels use tcgen05 / TMEM / TMA instructions of sm_100a) and the
# PyTorch headers.  No GPU is needed to build: nvcc cross-compiles.
set -e
cd "$(dirname "${BASH_SOURCE[0]}")"
NVCC_BIN="${NVCC:-$(command -v nvcc || echo /usr/local/cuda/bin/nvcc)}"
if [ ! -x "$NVCC_BIN" ]; then
    echo "error: nvcc not found (set NVCC or install the CUDA toolkit)" >&2
    exit 1
fi
echo "nvcc:    $("$NVCC_BIN" --version | grep release)"
echo "PyTorch: $(python -c 'import torch; print(torch.__version__)')"
NVCC="$NVCC_BIN" python build_ext.py "$@"
python -c "from kolmogorov_moe_architecture_b200.ops.loader import ext_available; print('extension present:', ext_available())"
