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


import contextlib
import threading

_state = threading.local()


@contextlib.contextmanager
def deferred_init():
    """Inside this block ``Linear`` layers are created without ``nn.Linear``'s default initialisation: the caller
    initialises every one of them afterwards (``MoETransformer`` applies normal(0, init_std) to all Linear
    weights and zeros the biases), so drawing the default values first is one wasted pass over every weight."""
    prev = getattr(_state, "defer", False)
    _state.defer = True
    try:
        yield
    finally:
        _state.defer = prev


class Linear(nn.Linear):
    def reset_parameters(self) -> None:
        if not getattr(_state, "defer", False):
            super().reset_parameters()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)

