"""Native grouped-SwiGLU interface (API of the reference's ``moe_arch/kernels/__init__.py``):
``grouped_swiglu_forward`` on expert-sorted rows with segment bounds, the differentiable
``grouped_swiglu_with_grad`` and ``is_kernel_available``.

The reference's CUDA kernel is a scalar one-thread-per-output loop without tensor cores, launched
once per expert after copying the segment bounds to the host, and has no backward
(reference: moe_arch/kernels/grouped_gemm.cu:129-257).  Here the same call runs the grouped
tcgen05 GEMM with the SwiGLU epilogue, reads the bounds on the device, and is differentiable.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops.loader import ext_available


def is_kernel_available() -> bool:
    return torch.cuda.is_available() and ext_available()


def grouped_swiglu_forward_pytorch(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends):
    out = torch.zeros_like(sorted_inputs)
    for e, (s, t) in enumerate(zip(seg_starts.tolist(), seg_ends.tolist())):
        if t > s:
            x = sorted_inputs[s:t]
            out[s:t] = (F.silu(x @ W1[e]) * (x @ W2[e])) @ W3[e]
    return out


def grouped_swiglu_with_grad(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts=None, seg_ends=None):
    """out[i] = SwiGLU_{expert(i)}(sorted_inputs[i]); differentiable in the inputs and the weights."""
    from .. import ops
    ids = sorted_expert_ids.view(-1, 1).long()
    ones = torch.ones(ids.shape, dtype=sorted_inputs.dtype, device=sorted_inputs.device)
    return ops.grouped_swiglu(sorted_inputs, W1, W2, W3, ids, ones)


def grouped_swiglu_forward_cuda(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends):
    with torch.no_grad():
        return grouped_swiglu_with_grad(sorted_inputs, W1, W2, W3, sorted_expert_ids)


def grouped_swiglu_forward(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends, use_cuda_kernel=True):
    if use_cuda_kernel and sorted_inputs.is_cuda and is_kernel_available():
        return grouped_swiglu_forward_cuda(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends)
    return grouped_swiglu_forward_pytorch(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends)


class GroupedSwiGLUFunction(torch.autograd.Function):
    """``GroupedSwiGLUFunction.apply(sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts, seg_ends)`` for
    callers of the reference's autograd wrapper (moe_arch/kernels/__init__.py:140-225, whose backward is a Python
    loop of seven matmuls per expert).  Forward and backward both run the differentiable grouped path of
    ``grouped_swiglu_with_grad``: the forward records that path's own graph, the backward asks it for the gradients
    of the inputs and the three weight stacks."""

    @staticmethod
    def forward(ctx, sorted_inputs, W1, W2, W3, sorted_expert_ids, seg_starts=None, seg_ends=None):
        with torch.enable_grad():
            leaves = [t.detach().requires_grad_(t.requires_grad) for t in (sorted_inputs, W1, W2, W3)]
            out = grouped_swiglu_with_grad(*leaves, sorted_expert_ids)
        ctx.leaves, ctx.out = leaves, out
        return out.detach()

    @staticmethod
    def backward(ctx, grad_output):
        need = [t for t in ctx.leaves if t.requires_grad]
        got = iter(torch.autograd.grad(ctx.out, need, grad_output) if need else ())
        grads = [next(got) if t.requires_grad else None for t in ctx.leaves]
        ctx.leaves = ctx.out = None
        return (*grads, None, None, None)
