"""FP8 layers (API of the reference's ``moe_arch/model/fp8_moe.py``): ``FP8Linear``,
``FP8GroupedExperts``, ``FP8MoELayer``, ``is_fp8_available``.

The reference simulates FP8 (per-tensor delayed scaling, clamp to +-448, bf16 multiply).  Here the
number format is real block-scaled MXFP8 (e4m3 values, 1x32 power-of-two scales, see
``ops/mxfp8.py``); unlike the reference the experts are also selectable from the model config
(``moe_dtype: mxfp8``).  State-dict names (``weight``, ``w1/w2/w3`` and the scale / amax-history
buffers) are kept so reference checkpoints load.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import eager
from ..ops.mxfp8 import grouped_swiglu_mxfp8, linear_mx
from .linear import Linear

FP8_E4M3 = torch.float8_e4m3fn
FP8_E5M2 = torch.float8_e5m2


def is_fp8_available() -> bool:
    """True on GPUs with fp8 tensor cores (sm_89, sm_90, sm_100 and later)."""
    if not torch.cuda.is_available():
        return False
    p = torch.cuda.get_device_properties(0)
    return p.major >= 9 or (p.major == 8 and p.minor >= 9)


class FP8Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype or torch.bfloat16))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype or torch.bfloat16)) if bias else None
        for n in ("input_scale", "weight_scale", "output_scale"):
            self.register_buffer(n, torch.tensor(1.0))
        self.register_buffer("input_amax_history", torch.zeros(16))
        self.register_buffer("weight_amax_history", torch.zeros(16))
        self.history_idx = 0
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_mx(x, self.weight, self.bias)


class FP8GroupedExperts(nn.Module):
    def __init__(self, n_experts: int, d_model: int, d_ff: int):
        super().__init__()
        self.n_experts, self.d_model, self.d_ff = n_experts, d_model, d_ff
        self.w1 = nn.Parameter(torch.empty(n_experts, d_model, d_ff, dtype=torch.bfloat16))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, d_ff, dtype=torch.bfloat16))
        self.w3 = nn.Parameter(torch.empty(n_experts, d_ff, d_model, dtype=torch.bfloat16))
        for n in ("w1_scale", "w2_scale", "w3_scale"):
            self.register_buffer(n, torch.ones(n_experts))
        self.register_buffer("input_scale", torch.tensor(1.0))
        for w in (self.w1, self.w2, self.w3):
            nn.init.uniform_(w, -1.0 / math.sqrt(w.shape[1]), 1.0 / math.sqrt(w.shape[1]))

    def forward(self, x: torch.Tensor, expert_indices: torch.Tensor, expert_weights: torch.Tensor) -> torch.Tensor:
        return grouped_swiglu_mxfp8(x, self.w1, self.w2, self.w3, expert_indices, expert_weights)


class FP8MoELayer(nn.Module):
    """Router ``Linear(d, E)`` (softmax, top-k, renormalise) + MXFP8 experts; aux = E * sum f_i P_i * 0.01."""

    def __init__(self, d_model: int, d_ff: int, n_experts: int, top_k: int = 2):
        super().__init__()
        self.d_model, self.d_ff, self.n_experts, self.top_k = d_model, d_ff, n_experts, top_k
        self.router = Linear(d_model, n_experts, bias=False)
        self.experts = FP8GroupedExperts(n_experts, d_model, d_ff)
        self.aux_loss = 0.0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = x.reshape(-1, self.d_model)
        logits = self.router(flat.to(self.router.weight.dtype))
        w, idx = eager.topk_softmax_route(logits, self.top_k)
        if self.training:
            self.aux_loss = eager.moe_aux_loss(logits, idx, self.n_experts, 0.01, 0.0)
        return self.experts(flat, idx, w.to(flat.dtype)).view(shape)


def benchmark_fp8_vs_bf16(n_experts: int = 16, d_model: int = 1024, d_ff: int = 2048, n_tokens: int = 8192,
                          top_k: int = 2, n_iters: int = 20, device=None):
    """Block-scaled fp8 experts against the same experts in bf16, forward and forward + backward (reference:
    moe_arch/model/fp8_moe.py:341-394, whose fp8 path is simulated in bf16).  Needs a GPU with the library loaded;
    returns the milliseconds per call, or None where fp8 is unavailable."""
    from ._bench import default_device, report, routed_inputs, time_ms
    from .sparse_moe import SparseGroupedExpertsPyTorch
    device = device or default_device()
    if not (str(device).startswith("cuda") and is_fp8_available()):
        print("block-scaled fp8 needs a GPU with this library's kernels: nothing to compare")
        return None
    x, idx, w = routed_inputs(n_tokens, d_model, n_experts, top_k, device, torch.bfloat16)
    bf16 = SparseGroupedExpertsPyTorch(n_experts, d_model, d_ff).to(device).bfloat16()
    fp8 = FP8GroupedExperts(n_experts, d_model, d_ff).to(device).bfloat16()
    with torch.no_grad():
        for a, b in zip(fp8.parameters(), bf16.parameters()):
            a.copy_(b)
    times = {}
    for name, mod in (("bf16", bf16), ("mxfp8", fp8)):
        with torch.no_grad():
            times[f"{name} forward"] = time_ms(lambda: mod(x, idx, w), device, iters=n_iters)
        xs = x.detach().requires_grad_(True)
        times[f"{name} forward+backward"] = time_ms(lambda: mod(xs, idx, w).sum().backward(), device, iters=n_iters)
    with torch.no_grad():
        rel = float((fp8(x, idx, w).float() - bf16(x, idx, w).float()).norm() / bf16(x, idx, w).float().norm())
    print(f"relative difference of the outputs: {rel:.4f}")
    return report(f"{n_experts} experts, d_model {d_model}, d_ff {d_ff}, {n_tokens} tokens, top-{top_k}", times,
                  "bf16 forward")
