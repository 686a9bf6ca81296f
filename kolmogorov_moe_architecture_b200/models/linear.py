"""``nn.Linear`` whose products run on this library's GEMM.

Same parameters, initialisation and state-dict keys as ``torch.nn.Linear`` (the reference builds
every projection from it: moe_arch/model/attention.py:53-56, ffn.py:44-64, mamba.py:30-52); only
``forward`` differs: bf16 CUDA inputs go to the tcgen05 kernel for y = x W^T, dx = dy W and
dW = dy^T x, everything else to ``F.linear``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class Linear(nn.Linear):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)
