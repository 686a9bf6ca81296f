"""MXFP8 (OCP microscaling) support: e4m3 values with one power-of-two (e8m0) scale per 32
consecutive elements along the reduction dimension.

``quantize_mx`` / ``dequantize_mx`` define the number format exactly (they are the oracle for
any kernel that consumes it); ``fake_quant_mx`` is the straight-through estimator used for
training; ``grouped_swiglu_mxfp8`` runs the expert FFN with every GEMM operand (activations and
weights, forward and backward) rounded to MXFP8 along its own reduction axis, accumulating in
fp32 on the tcgen05 bf16 path - the values that enter the tensor core are exactly the MXFP8
values, so the arithmetic matches a block-scaled fp8 MMA while the operand bandwidth does not yet
benefit.  The reference's "FP8" experts clamp to +-448 and multiply in bf16 without ever casting to
an fp8 dtype (reference: moe_arch/model/fp8_moe.py:247-266).
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
BLOCK = 32


def _block_view(x: torch.Tensor, dim: int):
    x = x.movedim(dim, -1)
    K = x.shape[-1]
    pad = (-K) % BLOCK
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
    return x.reshape(*x.shape[:-1], -1, BLOCK), K


def quantize_mx(x: torch.Tensor, dim: int = -1):
    """Returns (q: float8_e4m3fn with x's shape, scale_exp: int8 exponents, one per 32-block along ``dim``).
    scale = 2^(floor(log2(amax)) - 8), the OCP rule for an element type with emax = 8."""
    xb, K = _block_view(x.float(), dim)
    amax = xb.abs().amax(dim=-1, keepdim=True)
    exp = torch.floor(torch.log2(amax.clamp(min=2.0 ** -127))) - 8.0
    exp = exp.clamp(-127, 127)
    scale = torch.exp2(exp)
    q = (xb / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(*xb.shape[:-2], -1)[..., :K].movedim(-1, dim)
    return q, exp.squeeze(-1).to(torch.int8)


def dequantize_mx(q: torch.Tensor, scale_exp: torch.Tensor, dim: int = -1, dtype=torch.bfloat16) -> torch.Tensor:
    qb, K = _block_view(q.float(), dim)
    out = qb * torch.exp2(scale_exp.float()).unsqueeze(-1)
    return out.reshape(*qb.shape[:-2], -1)[..., :K].movedim(-1, dim).to(dtype)


class _FakeQuantMX(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        q, e = quantize_mx(x, dim)
        return dequantize_mx(q, e, dim, x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None


def fake_quant_mx(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Round to MXFP8 along ``dim`` and return in x's dtype; identity gradient."""
    return _FakeQuantMX.apply(x, dim)


def grouped_swiglu_mxfp8(x, w1, w2, w3, idx, weights, keep=None):
    """Expert FFN with MXFP8-rounded operands.  Reduction axes: x along d, w1/w2 along d (dim 1),
    the SwiGLU hidden along f, w3 along f (dim 1)."""
    from . import cuda_ops, eager
    xq = fake_quant_mx(x, -1)
    w1q, w2q, w3q = fake_quant_mx(w1, 1), fake_quant_mx(w2, 1), fake_quant_mx(w3, 1)
    if x.is_cuda and x.dtype == torch.bfloat16:
        return cuda_ops._GroupedSwiGLU.apply(xq, w1q.contiguous(), w2q.contiguous(), w3q.contiguous(), idx, weights, keep)
    return eager.grouped_swiglu(xq, w1q, w2q, w3q, idx, weights, keep)
