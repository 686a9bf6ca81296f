"""Causal GQA flash attention on CUDA tensors (tcgen05 kernels in csrc/attention.cu)."""
from __future__ import annotations

import math

import torch

from . import eager


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, doc_start):
        from . import cuda_ops
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse = torch.ops.kmoe.attn_fwd(q, k, v, scale, doc_start, cuda_ops.status_tensor(q.device))
        cuda_ops._count()
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale, ctx.doc_start = scale, doc_start
        return out

    @staticmethod
    def backward(ctx, d_out):
        from . import cuda_ops
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = torch.ops.kmoe.attn_bwd(q, k, v, out, d_out.contiguous(), lse, ctx.scale, ctx.doc_start,
                                             cuda_ops.status_tensor(q.device))
        cuda_ops._count(3)
        return dq, dk, dv, None, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              doc_start: torch.Tensor = None) -> torch.Tensor:
    """q (B,S,H,D); k, v (B,S,Hkv,D) -> (B,S,H,D).  bf16, D in {64, 128}, causal.  ``doc_start`` (B, S) int32:
    first position of the packed document containing each position - attention then stays inside documents."""
    from . import cuda_ops
    D = q.shape[-1]
    if not (causal and q.dtype == torch.bfloat16 and D in (64, 128)):
        cuda_ops._fallback("attention", f"dtype {q.dtype} head_dim {D} causal {causal}")
        mask = eager.doc_start_to_mask(doc_start, q.dtype) if doc_start is not None else None
        return eager.attention(q, k, v, causal, mask)
    if doc_start is not None:
        doc_start = doc_start.to(torch.int32).contiguous()
    return _FlashAttn.apply(q, k, v, 1.0 / math.sqrt(D), doc_start)
